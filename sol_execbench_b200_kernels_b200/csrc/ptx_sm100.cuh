// Thin wrappers over the sm_100a PTX this library is built from: mbarriers with
// bounded waits, TMA tiled loads/stores, tcgen05 (TMEM allocation, MMA issue,
// commit, accumulator loads) and the matching fences.  No CUTLASS / CuTe.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gu {

// ---------------------------------------------------------------------------
// Device status word: [0] first error code (0 = none), [1] detail.
// ---------------------------------------------------------------------------
__device__ unsigned int g_status[4];

// Every device-side wait gives up after this many nanoseconds (2 s unless gu_set_wait_limit_ns changed it).
__device__ unsigned long long g_wait_limit_ns = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// back-off inside a bounded spin: lets the other warps of the SM issue while this one polls
__device__ __forceinline__ void spin_backoff_ns(uint32_t ns) { asm volatile("nanosleep.u32 %0;" ::"r"(ns)); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
}

// ---------------------------------------------------------------------------
// Abort protocol.  A wait that runs out records (code, detail) in g_status and
// raises a CTA-wide flag in shared memory; from then on every wait in the CTA
// returns at once and the roles skip their device work but keep their loop
// structure, so all warps still meet at the same barriers and the CTA exits.
// ---------------------------------------------------------------------------
struct WaitCtx {
  uint32_t abort_addr;  // shared::cta address of the CTA's abort flag
  bool aborted;
  bool pair;            // CTA pair: a failing wait raises the other CTA's flag too (same offset, other rank)
  __device__ __forceinline__ bool raised() const {
    uint32_t v;
    asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(abort_addr) : "memory");
    return v != 0u;
  }
  __device__ __forceinline__ void fail(unsigned code, unsigned detail) {
    aborted = true;
    asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(abort_addr), "r"(1u) : "memory");
    if (pair) {
      asm volatile(
          "{\n\t.reg .b32 r, a;\n\t"
          "mov.u32 r, %%cluster_ctarank;\n\t"
          "xor.b32 r, r, 1;\n\t"
          "mapa.shared::cluster.u32 a, %0, r;\n\t"
          "st.shared::cluster.u32 [a], %1;\n\t}"
          ::"r"(abort_addr), "r"(1u)
          : "memory");
    }
    if (atomicCAS(&g_status[0], 0u, code) == 0u) g_status[1] = detail;
  }
};

// ---------------------------------------------------------------------------
// Range-checked debug build (-DGU_BOUNDS=1; never the shipped library): every
// computed TMA coordinate, global index and ring / accumulator stage index is
// tested against its extent before it is used; the first violation is recorded
// in the status word (code kStatusBounds, detail = site << 16 | block) and the
// access is skipped.  In the regular build the tests compile to nothing.
// ---------------------------------------------------------------------------
constexpr unsigned kStatusBounds = 0x42;
#ifdef GU_BOUNDS
__device__ __forceinline__ bool bounds_ok(bool cond, unsigned site) {
  if (!cond && atomicCAS(&g_status[0], 0u, kStatusBounds) == 0u) g_status[1] = (site << 16) | (blockIdx.x & 0xffffu);
  return cond;
}
#define GU_IN_RANGE(cond, site) ::gu::bounds_ok((cond), (site))
#else
#define GU_IN_RANGE(cond, site) true
#endif

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}
// Bounded wait.  Returns false (after recording `code`) if the phase did not
// complete within kWaitTimeoutNs, or at once if the CTA is already aborting.
__device__ __forceinline__ bool mbar_wait(WaitCtx& ctx, uint32_t bar, uint32_t parity, unsigned code) {
  if (ctx.aborted) return false;
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (ctx.raised()) {
        ctx.aborted = true;
        return false;
      }
      if ((it & 1023u) == 0u) {
        unsigned long long now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > g_wait_limit_ns) {
          ctx.fail(code, (code << 24) | (blockIdx.x & 0xffffffu));
          return false;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor, tiled, 2-D).  No cluster multicast anywhere.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// x = innermost coordinate (elements), y = row.  x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM allocation, fences, MMA, commit, loads
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128
// bytes (one 128-byte swizzle span) and whose 8-row groups are 1024 bytes apart:
//   [0,14) start address >> 4 | [16,30) leading byte offset >> 4 (unused for this
//   layout, 1) | [32,46) stride byte offset >> 4 (1024 -> 64) | [46,48) version 1 |
//   [61,64) layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor, kind::f8f6f4: D fp32 (bits 4-5 = 1), A and B e4m3
// (format 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, one thread issues.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives (count 1) once every MMA this thread issued before has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Waits for this thread's outstanding tcgen05.ld.  The loaded registers are
// threaded through as in/out operands so no use of them can be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// (no instruction: makes the registers of an earlier tcgen05.ld look written here, after the wait)
template <int N>
__device__ __forceinline__ void pin_regs(float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(r[i]));
}
template <int N>
__device__ __forceinline__ void tmem_ld_wait_pin(float* v) {
  tmem_ld_wait();
  pin_regs<N>(v);
}

// ---------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs, tcgen05 with cta_group::2).  The even CTA of a
// pair issues the MMAs for both; each CTA keeps its own 128 accumulator lanes in
// its own TMEM and stages its own token rows plus HALF of the weight rows.
// Barriers are always waited on locally; the signalling side reaches into the
// other CTA with shared::cluster addresses (mapa).  No multicast form is used.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// hardware barrier over all threads of the cluster (cannot time out: only placed where every thread arrives)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// Arrivals on a barrier of either CTA of the pair.  Relaxed: what they hand over lives in TMEM or is written by
// the async proxy (ordered by the tcgen05 fences and the barrier's transaction count), not in memory this thread
// wrote, and a release at cluster scope would make the thread wait for every load it still has in flight.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Plain (non-multicast) tiled load into THIS CTA's shared memory whose completion bytes are counted on a barrier
// that may live in the other CTA of the pair (`cluster_bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m, uint32_t cluster_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {  // same warp id in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {  // same warp id in both CTAs
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[256 rows: 128 per CTA] * B[N rows: N/2 per CTA]^T; issued by one thread of the even CTA.
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// `cluster_bar` (either CTA's barrier, shared::cluster address) gets one arrival once every pair MMA issued before
// by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}

// ---------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out = bf16( f32(bf16(silu(f32(bf16 gate)))) * f32(bf16 up) ): the three
// rounding boundaries of the reference epilogue, as a float holding a bf16 value.
__device__ __forceinline__ float swiglu_bf16(float gate_acc, float up_acc) {
  float g = bf16_round(gate_acc);
  float u = bf16_round(up_acc);
  float act = bf16_round(__fdividef(g, 1.0f + __expf(-g)));
  return act * u;  // caller rounds to bf16 when packing
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Same three rounding boundaries for two adjacent columns at once, with every
// bf16 rounding done by the packed two-value conversion (half the conversion
// instructions) and the widening back to fp32 by shifts.  Returns the two bf16
// outputs packed (.x in the low half).
// `gp` / `up`: two bf16-rounded gate / up values, packed (.x in the low half).
__device__ __forceinline__ uint32_t swiglu_packed_bf16x2(uint32_t gp, uint32_t up) {
  const float g0 = __uint_as_float(gp << 16), g1 = __uint_as_float(gp & 0xffff0000u);
  const float a0 = __fdividef(g0, 1.0f + __expf(-g0));
  const float a1 = __fdividef(g1, 1.0f + __expf(-g1));
  const uint32_t ap = pack_bf16x2(a0, a1);
  // bf16 x bf16 is exact in fp32, so the packed bf16 multiply (one rounding of the exact product) gives the bits of
  // "widen, multiply in fp32, round to bf16" with one instruction instead of five
  const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ap), *reinterpret_cast<const __nv_bfloat162*>(&up));
  return *reinterpret_cast<const uint32_t*>(&prod);
}
__device__ __forceinline__ uint32_t swiglu_bf16x2(float2 gate_acc, float2 up_acc) {
  return swiglu_packed_bf16x2(pack_bf16x2(gate_acc.x, gate_acc.y), pack_bf16x2(up_acc.x, up_acc.y));
}

}  // namespace gu
