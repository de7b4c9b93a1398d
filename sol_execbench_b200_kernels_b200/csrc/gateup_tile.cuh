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
// Two schedules.  Data-parallel (kStreamK = false): CTA c takes tiles c, c+G,
// c+2G, ... of an L2-friendly raster; right when the tile count fills the SMs for
// many rounds.  Stream-K (kStreamK = true): the (tile, K block) units are cut into
// G equal contiguous ranges, so a tile count that is not a multiple of the SM
// count (112 tiles, 152 tiles, ...) no longer leaves SMs idle for a whole round.
// A range that starts inside a tile publishes its fp32 running sums (128 values
// per consumer thread) and an epoch-stamped flag; the range that holds the
// tile's first K block adds the later ranges' sums in range order and finishes
// the tile.  Hand-offs are produced at the start of a range and consumed at the
// end of an earlier one, ranges are numbered against blockIdx so a CTA only
// waits for CTAs dispatched before it, and the wait is bounded.
//
// Single-projection mode (kSingle): the same kernel as a plain block-scaled GEMM,
// C = bf16(sum_kb scale_a * scale_b * (A_kb . B_kb^T)) — the building block the
// reference launches twice (kernel.py:487-488).  The two 128-row weight tiles of a
// K block are then two ADJACENT 128-column blocks of one B matrix (scale rows 2n
// and 2n+1), so a CTA tile is 128 x 256 outputs, and the epilogue is two bf16
// casts and two stores instead of SwiGLU.  Used for the MLP's down projection.
//
// FP8-output mode (kFp8Out): the SwiGLU result is re-quantised in the epilogue to e4m3 with one fp32 scale
// per token and 128 columns (amax / 448) — the tile is exactly one scale block wide, so the row maximum is
// the larger of two threads' maxima, exchanged through shared memory — and stored as e4m3 [M, N] plus
// scales [M, N/128]: the operand format of the next block-scaled GEMM (the down projection), so the bf16
// intermediate never reaches HBM either.  The bits equal quantising the bf16 result with the torch quantiser.
//
// Warp roles (12 warps, 3 warpgroups so register budgets can be moved):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (lane 0)
//   warps 2-3   idle (they only give their registers away)
//   warps 4-11  consumers: promotion + epilogue; warp w reads TMEM lanes
//               32*(w%4)..+31; warps 4-7 own output columns 0-63 of the tile,
//               warps 8-11 columns 64-127 (gate and up of the same columns).
#pragma once

#include <cuda_fp8.h>

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
  kWaitStreamFlag = 9, kWaitTileFlag = 10,
};

struct TileParams {
  const float* scale_x;     // [M, kb]
  const float* scale_gate;  // [nb, kb]
  const float* scale_up;    // [nb, kb]
  int m, kb;                // tokens, K / 128
  int num_m_blocks, num_n_blocks, num_tiles;
  int group_m;              // M blocks per raster group (keeps a group's X tiles L2-resident)
  int tile_begin;           // stream-K launch: covers tiles [tile_begin, tile_begin + num_tiles) of the raster
  // gather launch only: every output tile is stored into out_count buffers (one per rank of the box) at a
  // column offset, so the all-gather of a column-sharded result happens inside the epilogue
  int out_count;
  int out_rank;             // this rank's index among the out_count buffers
  int out_col0;
  int n_blocks128;          // single-projection and fp8-output launches: N / 128
  float* scale_out;         // fp8-output launch only: [M, N/128] scales of the re-quantised result
  // scatter launch only (row-parallel GEMM whose partial results are summed over the ranks): the token blocks
  // are owned by ranks in runs of `blocks_per_owner`; a tile goes to its owner's buffer, into the slot of the
  // sending rank (slot s starts at row s * slot_rows of that buffer)
  int blocks_per_owner;
  int slot_rows;
  // stream-K schedule only
  unsigned int* flags;      // [gridDim.x] epoch of the last call that filled slot i
  float* partials;          // [gridDim.x][32][256] float4: values 4i..4i+3 of consumer thread t at [i * 256 + t]
  unsigned int epoch;       // this call's stamp, never 0
  // extents of the destination for the range-checked debug build (0: not checked)
  int out_rows = 0, out_cols = 0;
};

// sites of the range-checked debug build (see GU_IN_RANGE)
enum : unsigned {
  kSiteTileLoad = 1, kSiteTileScale = 2, kSiteTileStage = 3, kSiteTileStore = 4, kSiteTileHandOff = 5, kSiteTileScaleOut = 6,
  kSitePairLoad = 17, kSitePairScale = 18, kSitePairStage = 19, kSitePairStore = 20, kSitePairScaleOut = 21, kSitePairHandOff = 22,
  kSiteStreamLoad = 33, kSiteStreamScale = 34, kSiteStreamStage = 35, kSiteStreamStore = 36, kSiteStreamHandOff = 37,
};

// TMA load coordinates of a K block: x = K offset (16-byte aligned, inside K), rows inside the padded row range
__device__ __forceinline__ bool load_coords_ok(int kb, int j, int row, int row_limit) {
  return j >= 0 && j < kb && ((j * kBlockK) & 15) == 0 && row >= 0 && row < row_limit && (row & 127) == 0;
}

constexpr uint32_t kTileFlagBytes = 4096;                       // hand-off flags at the start of the workspace
constexpr int kTileMaxGrid = 256;                               // workspace is sized for at most this many ranges
constexpr uint32_t kTilePartialFloats = 128 * 256;              // one tile's running sums

// One CTA's walk over its work: whole tiles (data-parallel) or the tile segments of a unit range (stream-K).
// Stream-K tile numbers are relative to TileParams::tile_begin.
template <bool kStreamK>
struct TileWalk {
  uint32_t u, u_end;  // stream-K: next unit and end of the range (the host keeps tiles * kb below 2^31)
  int tile, step;
  __device__ __forceinline__ TileWalk(const TileParams& p, int worker, int workers)
      : u(0), u_end(0), tile(worker), step(workers) {
    if constexpr (kStreamK) {
      const unsigned long long units = static_cast<unsigned long long>(p.num_tiles) * p.kb;
      const int range = workers - 1 - worker;  // reverse order: see the file comment
      u = static_cast<uint32_t>(units * range / workers);
      u_end = static_cast<uint32_t>(units * (range + 1) / workers);
    }
  }
  // next segment: tile index and K blocks [j_begin, j_end)
  __device__ __forceinline__ bool next(const TileParams& p, int& t, int& j_begin, int& j_end) {
    if constexpr (kStreamK) {
      if (u >= u_end) return false;
      t = static_cast<int>(u / static_cast<uint32_t>(p.kb));
      j_begin = static_cast<int>(u - static_cast<uint32_t>(t) * p.kb);
      const uint32_t e = min(static_cast<uint32_t>(t + 1) * p.kb, u_end);
      j_end = j_begin + static_cast<int>(e - u);
      u = e;
      return true;
    } else {
      if (tile >= p.num_tiles) return false;
      t = tile;
      j_begin = 0;
      j_end = p.kb;
      tile += step;
      return true;
    }
  }
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

// Up to one output descriptor per GPU of the box (the gather launch stores every tile to all of them).
struct PeerMaps {
  CUtensorMap m[8];
};

// The kernel body; `outs` points at the output descriptor(s) in kernel parameter space.
template <bool kStreamK, bool kGather, bool kSingle = false, bool kFp8Out = false, bool kScatter = false>
__device__ __forceinline__ void tile_kernel_body(const CUtensorMap& tm_x, const CUtensorMap& tm_gate,
                                                 const CUtensorMap& tm_up, const CUtensorMap* outs,
                                                 const TileParams& p) {
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
    if constexpr (kGather || kScatter) {
      for (int r = 0; r < p.out_count; ++r) tma_prefetch_desc(&outs[r]);
    } else {
      tma_prefetch_desc(&outs[0]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTileTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  WaitCtx ctx{abort_slot, false, false};

  if (warp < 4) {
    reg_dealloc<64>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      int stage = 0;
      uint32_t phase = 0;
      TileWalk<kStreamK> walk(p, blockIdx.x, gridDim.x);
      int tile, jb, je;
      while (walk.next(p, tile, jb, je)) {
        int mb, nb;
        tile_coords(p, kStreamK ? tile + p.tile_begin : tile, mb, nb);
        for (int j = jb; j < je; ++j) {
          bool ok = mbar_wait(ctx, bar_empty + 8 * stage, phase ^ 1u, kWaitTileEmpty);
          ok = ok && GU_IN_RANGE(stage >= 0 && stage < kTileStages, kSiteTileStage) &&
               GU_IN_RANGE(load_coords_ok(p.kb, j, mb * kTileM, p.num_m_blocks * kTileM) &&
                               load_coords_ok(p.kb, j, nb * kTileN, p.num_n_blocks * kTileN), kSiteTileLoad);
          if (ok) {
            const uint32_t full = bar_full + 8 * stage;
            const uint32_t dst = ring + stage * kTileStageBytes;
            mbar_arrive_expect_tx(full, kTileStageBytes);
            tma_load_2d(dst, &tm_x, full, j * kBlockK, mb * kTileM);
            if constexpr (kSingle) {  // two adjacent 128-row blocks of the one B matrix (rows past N read as zero)
              tma_load_2d(dst + kOperandTileBytes, &tm_gate, full, j * kBlockK, 2 * nb * kTileN);
              tma_load_2d(dst + 2 * kOperandTileBytes, &tm_gate, full, j * kBlockK, (2 * nb + 1) * kTileN);
            } else {
              tma_load_2d(dst + kOperandTileBytes, &tm_gate, full, j * kBlockK, nb * kTileN);
              tma_load_2d(dst + 2 * kOperandTileBytes, &tm_up, full, j * kBlockK, nb * kTileN);
            }
          }
          if (++stage == kTileStages) { stage = 0; phase ^= 1u; }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------- MMA issuer -------------------------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(kTileM, 2 * kTileN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      TileWalk<kStreamK> walk(p, blockIdx.x, gridDim.x);
      int tile, jb, je;
      while (walk.next(p, tile, jb, je)) {
        for (int j = jb; j < je; ++j) {
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

    if constexpr (!kStreamK) {
      int tile = blockIdx.x;
      int mb = 0, nb = 0;
      const float *sx_row = p.scale_x, *sg_row = p.scale_gate, *su_row = p.scale_up;
      float sx0 = 0.f, sg0 = 0.f, su0 = 0.f, sx1 = 0.f, sg1 = 0.f, su1 = 0.f;
      // first two K blocks' scales of a tile (fetched before the previous tile's epilogue)
      auto start_tile = [&](int t) {
        tile_coords(p, t, mb, nb);
        const int m_global = min(mb * kTileM + row, p.m - 1);
        sx_row = p.scale_x + static_cast<size_t>(m_global) * p.kb;
        if constexpr (kSingle) {
          sg_row = p.scale_gate + static_cast<size_t>(2 * nb) * p.kb;
          su_row = p.scale_gate + static_cast<size_t>(min(2 * nb + 1, p.n_blocks128 - 1)) * p.kb;
        } else {
          sg_row = p.scale_gate + static_cast<size_t>(nb) * p.kb;
          su_row = p.scale_up + static_cast<size_t>(nb) * p.kb;
        }
        const int w_blocks = kSingle ? p.n_blocks128 : p.num_n_blocks;
        (void)w_blocks;  // (only the range-checked build looks at it)
        if (!GU_IN_RANGE(m_global >= 0 && m_global < p.m && (sg_row - p.scale_gate) / p.kb < w_blocks &&
                             (su_row - (kSingle ? p.scale_gate : p.scale_up)) / p.kb < w_blocks, kSiteTileScale))
          return;
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

        if constexpr (kFp8Out) {
          // -------- epilogue with re-quantisation: SwiGLU, row amax over the tile's 128 columns, e4m3 + scale --------
          uint32_t o2[32];  // this thread's 64 bf16 outputs, packed in pairs
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            o2[i] = swiglu_bf16x2(g[i], u[i]);
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(o2[i] << 16)), fabsf(__uint_as_float(o2[i] & 0xffff0000u))));
          }
          if (store_leader) tma_store_wait_read0();  // the previous store has finished reading the staging tile
          float* row_max = reinterpret_cast<float*>(smem_gen + (out_stage - smem_base) + kTileOutHalfBytes);  // [2][128]
          row_max[half * 128 + row] = amax;
          named_bar_sync(3, 256);
          amax = fmaxf(amax, row_max[(half ^ 1) * 128 + row]);
          const float sc = fmaxf(amax, 1e-12f) / 448.0f;
          const float rc = __frcp_rn(sc);
          // 64 e4m3 of this half at bytes [64*half, 64*half+64) of the row's 128 bytes (128-byte swizzle)
          uint8_t* out_row = smem_gen + (out_stage - smem_base) + row * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {  // 4 chunks of 16 e4m3
            uint32_t w[4];
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              uint32_t word = 0;
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const uint32_t pr = o2[8 * c + 2 * k4 + e];
                const float a = __uint_as_float(pr << 16), b = __uint_as_float(pr & 0xffff0000u);
                const float qa0 = a * rc, qb0 = b * rc;  // correctly rounded a / sc, b / sc (exact-residual step)
                const float qa = fmaf(fmaf(-qa0, sc, a), rc, qa0), qb = fmaf(fmaf(-qb0, sc, b), rc, qb0);
                word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qa, qb), __NV_SATFINITE, __NV_E4M3))
                        << (16 * e);
              }
              // (the residual step turns a quotient of -0 into +0; the sources' sign bits — the high byte of each
              // bf16, gathered by one byte permute — put the sign of such a zero back)
              w[k4] = word | (__byte_perm(o2[8 * c + 2 * k4], o2[8 * c + 2 * k4 + 1], 0x7531) & 0x80808080u);
            }
            const int chunk = half * 4 + c;
            *reinterpret_cast<uint4*>(out_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (half == 0 && cur_mb * kTileM + row < p.m && GU_IN_RANGE(cur_nb >= 0 && cur_nb < p.n_blocks128, kSiteTileScaleOut))
            p.scale_out[static_cast<size_t>(cur_mb * kTileM + row) * p.n_blocks128 + cur_nb] = sc;
          fence_proxy_async_smem();
          named_bar_sync(3, 256);
          if (threadIdx.x == 128 && !ctx.aborted) {
            tma_store_2d(&outs[0], out_stage, cur_nb * kTileN, cur_mb * kTileM);
            tma_store_commit();
          }
        } else if constexpr (kSingle) {
          // -------- epilogue of the plain GEMM: two 128-column blocks, each cast to bf16 and stored --------
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            if (store_leader) tma_store_wait_read0();  // the previous store has finished reading the staging tile
            named_bar_sync(1 + half, 128);
            uint8_t* out_row = smem_gen + (out_half - smem_base) + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const float2* src = part == 0 ? g : u;
              uint4 q;
              q.x = pack_bf16x2(src[4 * c + 0].x, src[4 * c + 0].y);
              q.y = pack_bf16x2(src[4 * c + 1].x, src[4 * c + 1].y);
              q.z = pack_bf16x2(src[4 * c + 2].x, src[4 * c + 2].y);
              q.w = pack_bf16x2(src[4 * c + 3].x, src[4 * c + 3].y);
              *reinterpret_cast<uint4*>(out_row + ((c ^ (row & 7)) << 4)) = q;
            }
            fence_proxy_async_smem();
            named_bar_sync(1 + half, 128);
            if (store_leader && !ctx.aborted && 2 * cur_nb + part < p.n_blocks128) {
              if constexpr (kScatter) {
                // partial result of a row-parallel GEMM: plain TMA store into the owner rank's buffer (over
                // NVLink unless it is this rank), in the slot reserved for this rank; the owner sums the slots
                const int owner = cur_mb / p.blocks_per_owner;
                const int y = p.out_rank * p.slot_rows + (cur_mb - owner * p.blocks_per_owner) * kTileM;
                tma_store_2d(&outs[owner], out_half, (2 * cur_nb + part) * kTileN + half * 64, y);
              } else {
                tma_store_2d(&outs[0], out_half, (2 * cur_nb + part) * kTileN + half * 64, cur_mb * kTileM);
              }
              tma_store_commit();
            }
          }
        } else {
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
            if constexpr (kGather) {
              // Plain TMA stores, one per rank's buffer (own and peers' over NVLink); no load touches peer memory.
              // Destinations are visited in a rotation that differs per source rank and per CTA, so that at any
              // moment the box's ranks are writing to different peers instead of all to the same one.
              const int peers = p.out_count - 1;
              const int col = p.out_col0 + cur_nb * kTileN + half * 64;
              tma_store_2d(&outs[p.out_rank], out_half, col, cur_mb * kTileM);
              for (int i = 0; i < peers; ++i) {
                const int hop = 1 + (i + static_cast<int>(blockIdx.x) + cur_mb) % peers;
                tma_store_2d(&outs[(p.out_rank + hop) % p.out_count], out_half, col, cur_mb * kTileM);
              }
            } else if (GU_IN_RANGE(p.out_cols == 0 || (cur_nb * kTileN + half * 64 + 64 <= p.out_cols &&
                                                       cur_mb * kTileM >= 0 && cur_mb * kTileM < p.out_rows),
                                   kSiteTileStore)) {
              tma_store_2d(&outs[0], out_half, cur_nb * kTileN + half * 64, cur_mb * kTileM);
            }
            tma_store_commit();
          }
        }
        tile = next;
      }
    } else {
      // ---- stream-K schedule: the same arithmetic in the same block order, but walking tile segments.  It runs
      // where the op is HBM-bound or on the last partial round of tiles, so the partial is read in four
      // 32-column pieces through one small buffer; the registers that frees hold the segment bookkeeping. ----
      const int ctid = threadIdx.x - 128;  // 0..255
      const int ranges = gridDim.x;
      const int my_range = ranges - 1 - static_cast<int>(blockIdx.x);
      TileWalk<true> walk(p, blockIdx.x, gridDim.x);
      int tile, jb, je;
      while (walk.next(p, tile, jb, je)) {
        int mb, nb;
        tile_coords(p, tile + p.tile_begin, mb, nb);
        const int m_global = min(mb * kTileM + row, p.m - 1);
        const float* sx_row = p.scale_x + static_cast<size_t>(m_global) * p.kb;
        const float* sg_row = p.scale_gate + static_cast<size_t>(nb) * p.kb;
        const float* su_row = p.scale_up + static_cast<size_t>(nb) * p.kb;

        float2 g[32], u[32];  // 64 gate + 64 up running sums
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          g[i] = make_float2(0.f, 0.f);
          u[i] = make_float2(0.f, 0.f);
        }
        float sx_n = __ldg(sx_row + jb), sg_n = __ldg(sg_row + jb), su_n = __ldg(su_row + jb);
        for (int j = jb; j < je; ++j) {
          const float sgx = sx_n * sg_n;
          const float sux = sx_n * su_n;
          if (j + 1 < je) { sx_n = __ldg(sx_row + j + 1); sg_n = __ldg(sg_row + j + 1); su_n = __ldg(su_row + j + 1); }
          const float2 sg2v = make_float2(sgx, sgx);
          const float2 su2v = make_float2(sux, sux);
          const bool ok = mbar_wait(ctx, my_acc_full + 8 * acc, acc_phase, kWaitTileAccFull);
          tc_fence_after();
          const uint32_t t = lane_addr + acc * (2 * kTileN);
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // gate columns 0-31, 32-63, then up columns 0-31, 32-63
            float v[32];
            if (ok) {
              tmem_ld32(t + (q >> 1) * kTileN + (q & 1) * 32, v);
              tmem_ld_wait_pin<32>(v);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0.f;
            }
            if (q == 3) {  // last piece is in registers: hand the TMEM stage back
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(my_acc_empty + 8 * acc);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 pv = make_float2(v[2 * i], v[2 * i + 1]);
              if (q < 2) g[(q & 1) * 16 + i] = __ffma2_rn(pv, sg2v, g[(q & 1) * 16 + i]);
              else u[(q & 1) * 16 + i] = __ffma2_rn(pv, su2v, u[(q & 1) * 16 + i]);
            }
          }
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }

        if (jb != 0) {
          // started inside the tile: publish the running sums for the range that owns the tile's first K block
          float4* slot = reinterpret_cast<float4*>(p.partials + static_cast<size_t>(my_range) * kTilePartialFloats) + ctid;
          if (GU_IN_RANGE(my_range >= 0 && my_range < kTileMaxGrid && ctid >= 0 && ctid < 256, kSiteTileHandOff))
#pragma unroll
          for (int i = 0; i < 16; ++i) {  // 16-byte stores, consecutive threads 16 bytes apart
            __stcg(slot + i * 256, make_float4(g[2 * i].x, g[2 * i].y, g[2 * i + 1].x, g[2 * i + 1].y));
            __stcg(slot + (16 + i) * 256, make_float4(u[2 * i].x, u[2 * i].y, u[2 * i + 1].x, u[2 * i + 1].y));
          }
          __threadfence();
          named_bar_sync(3, 256);
          if (ctid == 0 && !ctx.aborted) st_release_gpu(p.flags + my_range, p.epoch);
          continue;
        }
        if (je < p.kb) {
          // owner of the tile's first K block: add the later ranges' sums, in range order
          const unsigned long long units = static_cast<unsigned long long>(p.num_tiles) * p.kb;
          const unsigned long long tile_end = static_cast<unsigned long long>(tile + 1) * p.kb;
          for (int rr = my_range + 1; rr < ranges && units * rr / ranges < tile_end; ++rr) {
            if (store_leader && !ctx.aborted) {
              unsigned long long t0 = 0;
              for (uint32_t it = 1; ld_acquire_gpu(p.flags + rr) != p.epoch; ++it) {
                spin_backoff_ns(64u);
                if ((it & 255u) == 0u) {
                  const unsigned long long now = globaltimer_ns();
                  if (t0 == 0) {
                    t0 = now;
                  } else if (now - t0 > g_wait_limit_ns || ctx.raised()) {
                    ctx.fail(kWaitTileFlag, (kWaitTileFlag << 24) | (blockIdx.x & 0xffffffu));
                    break;
                  }
                }
              }
            }
            named_bar_sync(1 + half, 128);
            if (!ctx.raised()) {
              const float4* slot =
                  reinterpret_cast<const float4*>(p.partials + static_cast<size_t>(rr) * kTilePartialFloats) + ctid;
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float4 a = __ldcg(slot + i * 256);
                const float4 b = __ldcg(slot + (16 + i) * 256);
                g[2 * i].x += a.x; g[2 * i].y += a.y; g[2 * i + 1].x += a.z; g[2 * i + 1].y += a.w;
                u[2 * i].x += b.x; u[2 * i].y += b.y; u[2 * i + 1].x += b.z; u[2 * i + 1].y += b.w;
              }
            }
          }
        }
        // -------- epilogue, as in the data-parallel schedule --------
        if (store_leader) tma_store_wait_read0();
        named_bar_sync(1 + half, 128);
        {
          uint8_t* out_row = smem_gen + (out_half - smem_base) + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
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
          tma_store_2d(&outs[0], out_half, nb * kTileN + half * 64, mb * kTileM);
          tma_store_commit();
        }
      }
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
    while (globaltimer_ns() - t0 < 200000ull) spin_backoff_ns(1000u);
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTileTmemCols);
}

template <bool kStreamK>
__global__ void __launch_bounds__(kTileThreads, 1)
gateup_tile_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                   const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_out,
                   const TileParams p) {
  tile_kernel_body<kStreamK, false>(tm_x, tm_gate, tm_up, &tm_out, p);
}

// Gate/up + SwiGLU with the result re-quantised to e4m3 + 1x128 scales in the epilogue; `tm_outq` describes
// the e4m3 [M, N] destination with 128-byte x 128-row boxes.
__global__ void __launch_bounds__(kTileThreads, 1)
gateup_tile_fp8out_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                          const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_outq,
                          const TileParams p) {
  tile_kernel_body<false, false, false, true>(tm_x, tm_gate, tm_up, &tm_outq, p);
}

// Plain block-scaled GEMM (single-projection mode), data-parallel schedule.
__global__ void __launch_bounds__(kTileThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_c, const TileParams p) {
  tile_kernel_body<false, false, true>(tm_a, tm_b, tm_b, &tm_c, p);
}

// Plain block-scaled GEMM whose output tiles are scattered to the ranks that own their token rows
// (see TileParams::blocks_per_owner): the compute half of a fused GEMM + reduce-scatter.
__global__ void __launch_bounds__(kTileThreads, 1)
blockwise_gemm_scatter_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                              const __grid_constant__ PeerMaps peers, const TileParams p) {
  tile_kernel_body<false, false, true, false, true>(tm_a, tm_b, tm_b, peers.m, p);
}

// Data-parallel schedule with the column all-gather fused into the epilogue (see TileParams::out_count).
__global__ void __launch_bounds__(kTileThreads, 1)
gateup_tile_gather_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                          const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ PeerMaps peers,
                          const TileParams p) {
  tile_kernel_body<false, true>(tm_x, tm_gate, tm_up, peers.m, p);
}

}  // namespace gu
