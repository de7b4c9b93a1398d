// Input projection of the Mamba mixer (problem 029):
//   projected[M, N] = bf16( hidden[M, K] . weight[N, K]^T + bias[N] ),  all operands bf16, fp32 accumulation,
// one rounding at the end (the reference's CUTLASS builder GEMM with a row-broadcast bias in the epilogue:
// kernels/029_mamba_conv1d_with_gating/kernel.cu:36-160, launched from kernel.cu:274-312).
//
// A persistent tcgen05 kernel, kind::f16 with bf16 operands.  The accumulator of a tile stays in TMEM over the whole
// K loop (nothing has to pass through registers per K block here, unlike the block-scaled FP8 kernels), TMEM holds
// two 256-column accumulators, and the epilogue of a tile runs on its own warps while the next tile's MMAs fill the
// other accumulator.
//
//   kPair = true   two CTAs on neighbouring SMs own a 256-row x 256-column tile: each stages its own 128 rows of
//                  `hidden` and HALF of the 256 weight rows of a K block (32 KiB per CTA and 64-wide K block), the
//                  even CTA issues cta_group::2 MMAs (M = 256, N = 256, K = 16) for both; each CTA finds its
//                  128 x 256 fp32 accumulator in its own TMEM.  Used for M > 128.
//   kPair = false  one CTA owns a 128-row x 256-column tile and stages all 256 weight rows (48 KiB per K block).
//                  Used for M <= 128, where the second CTA of a pair would have no rows.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM allocation and (in the even CTA) MMA issue, warps 2-5
// epilogue: a warp reads TMEM lanes 32 (w % 4) .. +31 in chunks of 64 columns, adds the bias in fp32, rounds to bf16
// into one of two 16 KiB staging tiles (128-byte rows, 16-byte chunks swizzled by the row) and one thread issues the
// TMA store of the chunk, so the store of a chunk overlaps the conversion of the next.
//
// Every wait is on a barrier of the waiting CTA and is bounded; the other CTA of a pair reaches it with
// shared::cluster addresses (remote mbarrier.arrive, TMA completion bytes, tcgen05.commit).  No multicast form.
#pragma once

#include "ptx_sm100.cuh"

namespace so {

using namespace gu;

constexpr int kPjThreads = 192;
constexpr int kPjTileM = 128;                 // rows per CTA
constexpr int kPjTileN = 256;                 // columns per tile
constexpr int kPjBlockK = 64;                 // bf16 per K block: one 128-byte swizzle span
constexpr uint32_t kPjATileBytes = kPjTileM * 128;
constexpr uint32_t kPjOutChunkBytes = kPjTileM * 128;   // 128 rows x 64 bf16
constexpr uint32_t kPjOutBytes = 2 * kPjOutChunkBytes;
constexpr uint32_t kPjTmemCols = 512;         // two 256-column fp32 accumulators

template <bool kPair>
struct PjCfg {
  static constexpr int b_rows = kPair ? 128 : 256;  // weight rows this CTA stages per K block
  static constexpr uint32_t stage_bytes = kPjATileBytes + b_rows * 128;
  static constexpr int stages = kPair ? 6 : 4;
  static constexpr uint32_t smem_bytes = stages * stage_bytes + kPjOutBytes + 256 /*barriers*/ + 1024 /*alignment*/;
  static constexpr int rows_per_tile = kPair ? 2 * kPjTileM : kPjTileM;
};

enum : unsigned { kWaitPjSlot = 40, kWaitPjFull = 41, kWaitPjAccFree = 42, kWaitPjAccFull = 43 };
// sites of the range-checked debug build (-DGU_BOUNDS=1, see GU_IN_RANGE)
enum : unsigned { kSitePjLoad = 49, kSitePjStage = 50, kSitePjStore = 51, kSitePjBias = 52, kSitePjTile = 53 };

struct ProjParams {
  const __nv_bfloat16* bias;  // [N]
  int m, n, kb;               // kb = ceil(K / 64)
  int m_tiles, n_tiles, num_tiles;
  int group_m;                // raster: tiles walk `group_m` row tiles at a time, row tile fastest
};

// Instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B bf16 (format 1 at bits 7-9 and 10-12), both
// K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
template <bool kPair>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// One lane of a converged warp polls; every lane gets the outcome.
__device__ __forceinline__ bool pj_wait_elected(WaitCtx& ctx, bool elected, uint32_t bar, uint32_t parity, unsigned code) {
  bool ok = true;
  if (elected) ok = mbar_wait(ctx, bar, parity, code);
  ok = __all_sync(0xffffffffu, ok);
  __syncwarp();
  return ok;
}

__device__ __forceinline__ void pj_tile_coords(const ProjParams& p, int tile, int& tm, int& tn) {
  const int per_group = p.group_m * p.n_tiles;
  const int group = tile / per_group;
  const int first = group * p.group_m;
  const int rows = min(p.group_m, p.m_tiles - first);
  const int within = tile - group * per_group;
  tm = first + within % rows;
  tn = within / rows;
}

template <bool kPair>
__device__ __forceinline__ void proj_gemm_body(const CUtensorMap& tm_a, const CUtensorMap& tm_w,
                                               const CUtensorMap& tm_out, const ProjParams& p) {
  using Cfg = PjCfg<kPair>;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern; both CTAs of a pair get the same offsets
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t ring = smem_base;
  const uint32_t stag = ring + Cfg::stages * Cfg::stage_bytes;
  const uint32_t bars = stag + kPjOutBytes;
  const uint32_t bar_full = bars;                             // [stages] pair: the even CTA's, 2 arrivals + both CTAs' bytes
  const uint32_t bar_empty = bar_full + 8 * Cfg::stages;      // [stages] one commit: the slot's MMAs have read it
  const uint32_t bar_acc_full = bar_empty + 8 * Cfg::stages;  // [2] one commit: the tile's accumulator is complete
  const uint32_t bar_acc_free = bar_acc_full + 16;            // [2] pair: the even CTA's; 4 epilogue warps per CTA
  const uint32_t tmem_slot = bar_acc_free + 16;
  const uint32_t abort_slot = tmem_slot + 4;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_gen = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;
  const int unit = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int units = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::stages; ++s) {
      mbar_init(bar_full + 8 * s, kPair ? 2 : 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(bar_acc_full + 8 * q, 1);
      mbar_init(bar_acc_free + 8 * q, kPair ? 8 : 4);
    }
    *abort_gen = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(tmem_slot, kPjTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kPjTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (kPair) cluster_sync_all();  // barriers and the abort flag of both CTAs exist before anything reaches across
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  WaitCtx ctx{abort_slot, false, kPair};

  if (warp == 0) {
    // ---------------- TMA producer: the whole warp walks the loop, one elected lane waits and issues ----------------
    const bool elected = elect_one() != 0u;
    const uint32_t full_base = kPair ? mapa_shared(bar_full, 0) : bar_full;
    uint32_t slots = 0;  // ring slots filled so far: stage = low part, barrier phase = the next bit
    for (int tile = unit; tile < p.num_tiles; tile += units) {
      int tm, tn;
      pj_tile_coords(p, tile, tm, tn);
      const int row0 = tm * Cfg::rows_per_tile + static_cast<int>(rank) * kPjTileM;
      const int wrow0 = tn * kPjTileN + static_cast<int>(rank) * Cfg::b_rows;  // (rank is 0 without pairs)
      for (int j = 0; j < p.kb; ++j, ++slots) {
        const uint32_t stage = slots % Cfg::stages, phase = (slots / Cfg::stages) & 1u;
        const bool ok = pj_wait_elected(ctx, elected, bar_empty + 8 * stage, phase ^ 1u, kWaitPjSlot);
        const uint32_t full = full_base + 8 * stage;
        const uint32_t dst = ring + stage * Cfg::stage_bytes;
        // (loads may start past the last row of a ragged tile, where they read zeros, but never before row 0, past the
        // padded row range, or at a K offset that is not 16-byte aligned)
        if (ok && elected && GU_IN_RANGE(stage < static_cast<uint32_t>(Cfg::stages), kSitePjStage) &&
            GU_IN_RANGE(tm >= 0 && tm < p.m_tiles && tn >= 0 && tn < p.n_tiles, kSitePjTile) &&
            GU_IN_RANGE(j >= 0 && j < p.kb && ((j * kPjBlockK * 2) & 15) == 0 && row0 >= 0 &&
                            row0 < p.m_tiles * Cfg::rows_per_tile && wrow0 >= 0 && wrow0 < p.n_tiles * kPjTileN,
                        kSitePjLoad)) {
          // rows past M / N and columns past K read as zero
          if constexpr (kPair) {
            mbar_arrive_expect_tx_cluster(full, Cfg::stage_bytes);
            tma_load_2d_pair(dst, &tm_a, full, j * kPjBlockK, row0);
            tma_load_2d_pair(dst + kPjATileBytes, &tm_w, full, j * kPjBlockK, wrow0);
          } else {
            mbar_arrive_expect_tx(full, Cfg::stage_bytes);
            tma_load_2d(dst, &tm_a, full, j * kPjBlockK, row0);
            tma_load_2d(dst + kPjATileBytes, &tm_w, full, j * kPjBlockK, wrow0);
          }
        }
        __syncwarp();
      }
    }
    // the last commits into this CTA's ring barriers must have landed before the CTA may go away
    for (int s = 0; s < Cfg::stages; ++s, ++slots)
      pj_wait_elected(ctx, elected, bar_empty + 8 * (slots % Cfg::stages), ((slots / Cfg::stages) & 1u) ^ 1u, kWaitPjSlot);
  } else if (warp == 1) {
    if (rank == 0) {
      // ---------------- MMA issuer: the whole warp walks the loop, one elected lane waits and issues ----------------
      const bool elected = elect_one() != 0u;
      constexpr uint32_t idesc = umma_idesc_bf16_f32(Cfg::rows_per_tile, kPjTileN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t empty_odd = kPair ? mapa_shared(bar_empty, 1) : 0u;
      const uint32_t acc_full_odd = kPair ? mapa_shared(bar_acc_full, 1) : 0u;
      const uint64_t adesc0 = umma_desc_k_sw128(ring);
      const uint64_t bdesc0 = umma_desc_k_sw128(ring + kPjATileBytes);
      uint32_t blocks = 0, tiles_done = 0;
      for (int tile = unit; tile < p.num_tiles; tile += units, ++tiles_done) {
        const uint32_t acc = tiles_done & 1u, acc_phase = (tiles_done >> 1) & 1u;
        const uint32_t d = tmem_u + acc * kPjTileN;
        bool ok = pj_wait_elected(ctx, elected, bar_acc_free + 8 * acc, acc_phase ^ 1u, kWaitPjAccFree);
        for (int j = 0; j < p.kb; ++j, ++blocks) {
          const uint32_t stage = blocks % Cfg::stages, phase = (blocks / Cfg::stages) & 1u;
          const uint64_t adesc = adesc0 + stage * (Cfg::stage_bytes >> 4);
          const uint64_t bdesc = bdesc0 + stage * (Cfg::stage_bytes >> 4);
          ok = pj_wait_elected(ctx, elected, bar_full + 8 * stage, phase, kWaitPjFull) && ok;
          if (ok && elected) {
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kPjBlockK / 16; ++kk)  // 16 bf16 along K inside the swizzle span: +2 in the address field
              umma_bf16<kPair>(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (j > 0 || kk > 0) ? 1u : 0u);
            if constexpr (kPair) {
              umma_commit_pair(bar_empty + 8 * stage);
              umma_commit_pair(empty_odd + 8 * stage);
              if (j + 1 == p.kb) {
                umma_commit_pair(bar_acc_full + 8 * acc);
                umma_commit_pair(acc_full_odd + 8 * acc);
              }
            } else {
              umma_commit(bar_empty + 8 * stage);
              if (j + 1 == p.kb) umma_commit(bar_acc_full + 8 * acc);
            }
          }
          __syncwarp();
        }
      }
      // the last hand-backs (the odd CTA's among them) must have landed here before this CTA may go away
      for (uint32_t b = tiles_done; b < tiles_done + 2; ++b)
        pj_wait_elected(ctx, elected, bar_acc_free + 8 * (b & 1u), ((b >> 1) & 1u) ^ 1u, kWaitPjAccFree);
    }
  } else {
    // -------------------------------- epilogue (warps 2-5) ---------------------------------
    const int et = static_cast<int>(threadIdx.x) - 64;  // 0 .. 127
    const int quarter = warp & 3;                        // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;                 // row inside this CTA's 128
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t acc_free = kPair ? mapa_shared(bar_acc_free, 0) : bar_acc_free;
    uint8_t* stag_gen = smem_gen + (stag - smem_base);
    uint32_t tiles_done = 0;
    for (int tile = unit; tile < p.num_tiles; tile += units, ++tiles_done) {
      int tm, tn;
      pj_tile_coords(p, tile, tm, tn);
      const int row0 = tm * Cfg::rows_per_tile + static_cast<int>(rank) * kPjTileM;
      const int col0 = tn * kPjTileN;
      const uint32_t acc = tiles_done & 1u, acc_phase = (tiles_done >> 1) & 1u;
      const bool ok = pj_wait_elected(ctx, lane == 0, bar_acc_full + 8 * acc, acc_phase, kWaitPjAccFull);
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < kPjTileN / 64; ++c) {
        const int colc = col0 + 64 * c;
        float v[64];
        tmem_ld32(lane_addr + acc * kPjTileN + 64 * c, v);
        tmem_ld32(lane_addr + acc * kPjTileN + 64 * c + 32, v + 32);
        uint4 bq[8];  // this chunk's 64 bias values (the same for every row: broadcast loads)
#pragma unroll
        for (int q = 0; q < 8; ++q)
          bq[q] = (colc + 8 * q < p.n && GU_IN_RANGE(colc + 8 * q >= 0 && colc + 8 * q + 8 <= p.n, kSitePjBias))
                      ? __ldg(reinterpret_cast<const uint4*>(p.bias + colc + 8 * q))
                      : make_uint4(0, 0, 0, 0);
        tmem_ld_wait_pin<64>(v);
        if (c + 1 == kPjTileN / 64) {
          // the whole accumulator is in registers or stored: hand it back to the issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) mbar_arrive_cluster(acc_free + 8 * acc);
            else mbar_arrive(acc_free + 8 * acc);
          }
        }
        // the staging tile of this chunk was last read by the store issued two chunks ago
        if (et == 0) tma_store_wait_read1();
        named_bar_sync(1, 128);
        uint8_t* dst_row = stag_gen + (c & 1) * kPjOutChunkBytes + row * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t bw[4] = {bq[q].x, bq[q].y, bq[q].z, bq[q].w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float b_lo = __uint_as_float(bw[i] << 16), b_hi = __uint_as_float(bw[i] & 0xffff0000u);
            o[i] = pack_bf16x2(v[8 * q + 2 * i] + b_lo, v[8 * q + 2 * i + 1] + b_hi);
          }
          *reinterpret_cast<uint4*>(dst_row + ((q ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        // (a store may reach past the last row or column, where it is clipped, but starts inside the tensor)
        if (et == 0) {
          if (ok && !ctx.aborted && row0 < p.m && colc < p.n &&
              GU_IN_RANGE(row0 >= 0 && colc >= 0 && ((colc * 2) & 15) == 0, kSitePjStore))
            tma_store_2d(&tm_out, stag + (c & 1) * kPjOutChunkBytes, colc, row0);  // rows past M, columns past N are clipped
          // one group per chunk, also when the chunk lies outside the tensor and nothing is stored (an empty group):
          // "all groups but the newest have been read" above then always means "the store two chunks back has"
          tma_store_commit();
        }
      }
    }
    if (et == 0) tma_store_wait_all0();
  }

  // ------------------------------- teardown --------------------------------
  if (*abort_gen) {
    // give copies that were already in flight time to land before shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) spin_backoff_ns(1000u);
  }
  tc_fence_before();
  __syncwarp();
  if constexpr (kPair) cluster_sync_all();  // neither CTA leaves while the other may still reach into it
  else __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, kPjTmemCols);
    else tmem_dealloc(tmem_base, kPjTmemCols);
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPjThreads, 1)
proj_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_out, const ProjParams p) {
  proj_gemm_body<true>(tm_a, tm_w, tm_out, p);
}

__global__ void __launch_bounds__(kPjThreads, 1)
proj_gemm_lone_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_out, const ProjParams p) {
  proj_gemm_body<false>(tm_a, tm_w, tm_out, p);
}

}  // namespace so
