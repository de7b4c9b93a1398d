// Persistent tile kernel for the FP8 gate/up projection with fused SwiGLU.
//
// One CTA owns a 128-token x 128-column output tile and computes BOTH
// projections for it: per 128-wide K block it loads one X tile and the matching
// gate and up weight tiles (three plain TMA boxes, 48 KiB), and a single
// tcgen05.mma sequence with N = 256 leaves the gate partial in TMEM columns
// [0,128) and the up partial in [128,256) of a double-buffered accumulator.
// (One N = 256 instruction stream, not two of N = 128: the MMA is limited by
// shared-memory operand reads, and the narrower form reads the X tile twice.)
// Eight consumer warps read each partial out of TMEM, apply
// scale_x[m, kb] * scale_w[n/128, kb] and add it to fp32 running sums they keep
// in registers (block order ascending, as the reference's promotion loop does:
// variants/cute_fused_v1/blockwise_gemm_fused.py:1817-1823).  The same threads
// finish the tile: bf16 rounding of gate and up, SiLU, product, bf16 cast, a
// 128-byte-swizzled staging tile in shared memory and a TMA store.  Gate and up
// never reach HBM, X is read once per tile, and no CTA talks to another.
//
// Warp roles (12 warps, 3 warpgroups so register budgets can be moved):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (lane 0)
//   warps 2-3   idle (they only give their registers away)
//   warps 4-11  consumers: promotion + epilogue; warp w reads TMEM lanes
//               32*(w%4)..+31; warps 4-7 own output columns 0-63 of the tile,
//               warps 8-11 columns 64-127 (gate and up of the same columns).
#pragma once

#include "ptx_sm100.cuh"

namespace gu {

constexpr int kTileM = 128;         // tokens per tile (MMA M)
constexpr int kTileN = 128;         // output columns per tile; MMA N = 2 * kTileN
constexpr int kBlockK = 128;        // K elements (= bytes) per pipeline step, one scale block
constexpr int kTileStages = 4;      // shared-memory ring depth
constexpr int kTileThreads = 384;
constexpr uint32_t kOperandTileBytes = 128 * 128;            // 16 KiB: 128 rows x 128 B
constexpr uint32_t kTileStageBytes = 3 * kOperandTileBytes;  // X, gate, up
constexpr uint32_t kTileOutHalfBytes = 128 * 128;            // 128 rows x 64 bf16
constexpr uint32_t kTileSmemBytes =
    kTileStages * kTileStageBytes + 2 * kTileOutHalfBytes + 256 /*barriers*/ + 1024 /*alignment slack*/;
constexpr uint32_t kTileTmemCols = 512;  // 2 accumulator stages x 256 columns

// wait ids reported in the status word
enum : unsigned {
  kWaitTileEmpty = 1, kWaitTileFull = 2, kWaitTileAccEmpty = 3, kWaitTileAccFull = 4,
  kWaitStreamEmpty = 5, kWaitStreamFull = 6, kWaitStreamAccEmpty = 7, kWaitStreamAccFull = 8,
  kWaitStreamFlag = 9,
};

struct TileParams {
  const float* scale_x;     // [M, kb]
  const float* scale_gate;  // [nb, kb]
  const float* scale_up;    // [nb, kb]
  int m, kb;                // tokens, K / 128
  int num_m_blocks, num_n_blocks, num_tiles;
  int group_m;              // M blocks per raster group (keeps a group's X tiles L2-resident)
};

__device__ __forceinline__ void tile_coords(const TileParams& p, int tile, int& mb, int& nb) {
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = tile / per_group;
  const int r = tile - g * per_group;
  const int first_m = g * p.group_m;
  const int gm = min(p.group_m, p.num_m_blocks - first_m);
  nb = r / gm;
  mb = first_m + (r - nb * gm);
}

__global__ void __launch_bounds__(kTileThreads, 1)
gateup_tile_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                   const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_out,
                   const TileParams p) {
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t ring = smem_base;
  const uint32_t out_stage = smem_base + kTileStages * kTileStageBytes;
  const uint32_t bars = out_stage + 2 * kTileOutHalfBytes;
  const uint32_t bar_full = bars;                         // [kTileStages]
  const uint32_t bar_empty = bars + 8 * kTileStages;      // [kTileStages]
  const uint32_t bar_acc_full = bars + 16 * kTileStages;  // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;       // [2]
  const uint32_t tmem_slot = bar_acc_empty + 16;
  const uint32_t abort_slot = tmem_slot + 4;
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_gen = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTileStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 8);  // one arrival per consumer warp
    }
    *abort_gen = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_gate);
    tma_prefetch_desc(&tm_up);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTileTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  WaitCtx ctx{abort_gen, false};

  if (warp < 4) {
    reg_dealloc<64>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        int mb, nb;
        tile_coords(p, tile, mb, nb);
        for (int j = 0; j < p.kb; ++j) {
          const bool ok = mbar_wait(ctx, bar_empty + 8 * stage, phase ^ 1u, kWaitTileEmpty);
          if (ok) {
            const uint32_t full = bar_full + 8 * stage;
            const uint32_t dst = ring + stage * kTileStageBytes;
            mbar_arrive_expect_tx(full, kTileStageBytes);
            tma_load_2d(dst, &tm_x, full, j * kBlockK, mb * kTileM);
            tma_load_2d(dst + kOperandTileBytes, &tm_gate, full, j * kBlockK, nb * kTileN);
            tma_load_2d(dst + 2 * kOperandTileBytes, &tm_up, full, j * kBlockK, nb * kTileN);
          }
          if (++stage == kTileStages) { stage = 0; phase ^= 1u; }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------- MMA issuer -------------------------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(kTileM, 2 * kTileN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        for (int j = 0; j < p.kb; ++j) {
          bool ok = mbar_wait(ctx, bar_acc_empty + 8 * acc, acc_phase ^ 1u, kWaitTileAccEmpty);
          ok = mbar_wait(ctx, bar_full + 8 * stage, phase, kWaitTileFull) && ok;
          if (ok) {
            tc_fence_after();
            const uint32_t a_addr = ring + stage * kTileStageBytes;
            const uint64_t adesc = umma_desc_k_sw128(a_addr);
            const uint64_t bdesc = umma_desc_k_sw128(a_addr + kOperandTileBytes);
            const uint32_t d = tmem_base + acc * (2 * kTileN);
#pragma unroll
            for (int kk = 0; kk < kBlockK / 32; ++kk) {
              // 32 e4m3 = 32 bytes along K inside the swizzle span: +2 in the (>>4) address field
              umma_f8(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
            }
            umma_commit(bar_empty + 8 * stage);   // smem slot reusable once these MMAs have read it
            umma_commit(bar_acc_full + 8 * acc);  // partial complete in TMEM
          }
          if (++stage == kTileStages) { stage = 0; phase ^= 1u; }
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    reg_alloc<216>();
    // ------------------------------- consumers --------------------------------
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;      // which 64 output columns
    const int row = quarter * 32 + lane;   // token row inside the tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    const uint32_t out_half = out_stage + half * kTileOutHalfBytes;
    const uint32_t my_acc_full = bar_acc_full;
    const uint32_t my_acc_empty = bar_acc_empty;
    const bool store_leader = ((threadIdx.x - 128) & 127) == 0;
    int acc = 0;
    uint32_t acc_phase = 0;

    int tile = blockIdx.x;
    int mb = 0, nb = 0;
    const float *sx_row = p.scale_x, *sg_row = p.scale_gate, *su_row = p.scale_up;
    float sx0 = 0.f, sg0 = 0.f, su0 = 0.f, sx1 = 0.f, sg1 = 0.f, su1 = 0.f;
    // first two K blocks' scales of a tile (fetched before the previous tile's epilogue)
    auto start_tile = [&](int t) {
      tile_coords(p, t, mb, nb);
      const int m_global = min(mb * kTileM + row, p.m - 1);
      sx_row = p.scale_x + static_cast<size_t>(m_global) * p.kb;
      sg_row = p.scale_gate + static_cast<size_t>(nb) * p.kb;
      su_row = p.scale_up + static_cast<size_t>(nb) * p.kb;
      sx0 = __ldg(sx_row); sg0 = __ldg(sg_row); su0 = __ldg(su_row);
      if (p.kb > 1) { sx1 = __ldg(sx_row + 1); sg1 = __ldg(sg_row + 1); su1 = __ldg(su_row + 1); }
    };
    if (tile < p.num_tiles) start_tile(tile);

    while (tile < p.num_tiles) {
      float2 g[32], u[32];  // 64 gate + 64 up running sums
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        g[i] = make_float2(0.f, 0.f);
        u[i] = make_float2(0.f, 0.f);
      }

      for (int j = 0; j < p.kb; ++j) {
        // scales are fetched two K blocks ahead of their use
        float sx2 = 0.f, sg2 = 0.f, su2 = 0.f;
        if (j + 2 < p.kb) { sx2 = __ldg(sx_row + j + 2); sg2 = __ldg(sg_row + j + 2); su2 = __ldg(su_row + j + 2); }
        const float sgx = sx0 * sg0;
        const float sux = sx0 * su0;
        const float2 sg2v = make_float2(sgx, sgx);
        const float2 su2v = make_float2(sux, sux);

        const bool ok = mbar_wait(ctx, my_acc_full + 8 * acc, acc_phase, kWaitTileAccFull);
        tc_fence_after();
        float v[64];
        if (ok) {
          const uint32_t t = lane_addr + acc * (2 * kTileN);
          tmem_ld32(t, v);
          tmem_ld32(t + 32, v + 32);
          tmem_ld_wait_pin<64>(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = __ffma2_rn(make_float2(v[2 * i], v[2 * i + 1]), sg2v, g[i]);
          tmem_ld32(t + kTileN, v);
          tmem_ld32(t + kTileN + 32, v + 32);
          tmem_ld_wait_pin<64>(v);
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = 0.f;
        }
        // the partial is in registers: hand the TMEM stage back before the last FMAs
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(my_acc_empty + 8 * acc);
#pragma unroll
        for (int i = 0; i < 32; ++i) u[i] = __ffma2_rn(make_float2(v[2 * i], v[2 * i + 1]), su2v, u[i]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        sx0 = sx1; sg0 = sg1; su0 = su1;
        sx1 = sx2; sg1 = sg2; su1 = su2;
      }

      // next tile's coordinates and first scales, so their latency hides under the epilogue
      const int cur_mb = mb, cur_nb = nb;
      const int next = tile + gridDim.x;
      if (next < p.num_tiles) start_tile(next);

      // -------- epilogue: SwiGLU in registers, swizzled staging tile, TMA store --------
      if (store_leader) tma_store_wait_read0();  // previous tile's store has finished reading the staging tile
      named_bar_sync(1 + half, 128);
      {
        uint8_t* out_row = smem_gen + (out_half - smem_base) + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 8 chunks of 8 bf16 = 16 bytes
          uint4 q;
          q.x = swiglu_bf16x2(g[4 * c + 0], u[4 * c + 0]);
          q.y = swiglu_bf16x2(g[4 * c + 1], u[4 * c + 1]);
          q.z = swiglu_bf16x2(g[4 * c + 2], u[4 * c + 2]);
          q.w = swiglu_bf16x2(g[4 * c + 3], u[4 * c + 3]);
          *reinterpret_cast<uint4*>(out_row + ((c ^ (row & 7)) << 4)) = q;
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1 + half, 128);
      if (store_leader && !ctx.aborted) {
        tma_store_2d(&tm_out, out_half, cur_nb * kTileN + half * 64, cur_mb * kTileM);
        tma_store_commit();
      }
      tile = next;
    }
    if (store_leader) tma_store_wait_all0();
  }

  // ------------------------------- teardown --------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_gen) {
    // give copies that were already in flight time to land before shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTileTmemCols);
}

}  // namespace gu
