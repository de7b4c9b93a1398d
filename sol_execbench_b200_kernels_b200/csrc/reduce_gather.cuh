// Second half of the fused row-parallel GEMM + all-reduce: every rank owns a run of token rows; its buffer
// holds one bf16 partial result per sending rank (slot s = rows [s * slot_rows, (s+1) * slot_rows)).  This
// kernel adds the slots in rank order in fp32 (a fixed order: reproducible), rounds once to bf16 and writes
// the reduced rows into EVERY rank's full result at this rank's row offset — plain 16-byte stores, 512
// contiguous bytes per warp, to local memory and over NVLink to the peers.  Pure streaming, no loads from
// peer memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace gu {

struct ReduceGatherParams {
  const uint4* slots;       // this rank's [world][slot_rows][h] bf16, as 16-byte words
  uint4* outputs[8];        // every rank's [M][h] bf16 result buffer, as mapped into this process; null = skip
  long long words_per_slot; // slot_rows * h / 8
  long long out_word0;      // rank * slot_rows * h / 8: where this rank's rows start in a result buffer
  int world;
};

__global__ void __launch_bounds__(256) reduce_gather_kernel(const ReduceGatherParams p) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.words_per_slot; i += stride) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s >= p.world) break;
      const uint4 w = __ldcs(p.slots + s * p.words_per_slot + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 r;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
#pragma unroll
    for (int d = 0; d < 8; ++d)  // unrolled so that the pointer table stays in the parameter space
      if (d < p.world && p.outputs[d] != nullptr) p.outputs[d][p.out_word0 + i] = r;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Cross-rank barrier of one box, on the stream: every rank stamps its slot in every rank's flag array (plain
// stores, local and over NVLink) with this call's epoch and then polls ITS OWN array until every slot carries
// that epoch.  No load touches peer memory, and the wait is bounded: after `limit_ns` it records
// (GU_ETIMEOUT, wait id 20, missing rank) in the status word and the kernel returns, so a rank that never
// arrives costs its peers the time limit and an error code, not a hung GPU.
// Flag array of a rank (64 words, zeroed once before first use): [0, 8) arrival stamps by rank, [16] the number
// of barriers this rank has passed.  All ranks call the barrier the same number of times, so the counters agree.
// ---------------------------------------------------------------------------------------------------------
constexpr unsigned kWaitPeerBarrier = 20;
constexpr int kPeerFlagWords = 64;

struct PeerBarrierParams {
  unsigned int* flags[8];  // every rank's flag array as mapped into this process
  int world, rank;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrierParams p) {
  const int t = threadIdx.x;
  unsigned int* mine = p.flags[p.rank];
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(mine + 16) + 1u;
  __syncwarp();
  if (t < p.world) {
    // everything this rank's earlier kernels on the stream wrote (to any rank) is visible before the stamp is
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[t] + p.rank), "r"(epoch) : "memory");
    unsigned long long t0 = 0;
    for (unsigned int it = 1;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + t) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;  // (a peer may already be one barrier ahead)
      if ((it & 63u) == 0u) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > p.limit_ns) {
          if (atomicCAS(&g_status[0], 0u, kWaitPeerBarrier) == 0u)
            g_status[1] = (kWaitPeerBarrier << 24) | static_cast<unsigned int>(t);
          break;
        }
        spin_backoff_ns(200u);
      }
    }
  }
  __syncwarp();
  if (t == 0) *reinterpret_cast<volatile unsigned int*>(mine + 16) = epoch;
}

}  // namespace gu
