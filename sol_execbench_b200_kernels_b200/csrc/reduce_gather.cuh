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

}  // namespace gu
