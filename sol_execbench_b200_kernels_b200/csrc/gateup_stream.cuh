// Weight-streaming kernel for decode-sized token counts (M <= 64).
//
// With a handful of tokens the op is a pure read of both weight matrices, so the
// operands swap sides: a 128-row weight tile is the MMA "M" operand and the
// (padded) token block is the MMA "N" operand.  Each work unit is one 128 x 128
// K block of one output column block: a gate tile, an up tile (16 KiB each) and
// the small X tile, delivered by TMA into a deep shared-memory ring; two short
// tcgen05.mma sequences leave gate^T and up^T partials ([128 weight rows] x
// [MPAD tokens]) side by side in TMEM.  Four consumer warps — one thread per
// output column — read them, apply scale_x[t, kb] * scale_w[n/128, kb] and keep
// fp32 running sums per token in registers.
//
// Stream-K: the (column block, K block) units are numbered column-block-major
// and cut into gridDim.x equal contiguous ranges, one per CTA, so every SM
// streams the same number of weight bytes whatever N/128 is.  A range that
// starts in the middle of a column block hands its partial sums to the CTA that
// owns the block's first K block through a global scratch slot and a flag; that
// owner adds the partials in range order (a fixed order, so results are
// reproducible) and then applies SwiGLU and stores.  The hand-off is produced
// at the START of the later range and consumed at the END of the earlier one,
// so nobody waits in steady state; the wait is bounded all the same.
//
// Warps: 0 TMA producer, 1 TMEM allocation + MMA issue, 2-5 consumers.
#pragma once

#include "gateup_tile.cuh"

namespace gu {

constexpr int kStreamThreads = 192;
constexpr int kStreamAccStages = 4;
constexpr int kStreamMaxStages = 8;
constexpr uint32_t kStreamFlagBytes = 4096;  // up to 1024 hand-off flags at the start of the workspace
constexpr int kStreamMaxGrid = 256;          // workspace is sized for at most this many ranges

struct StreamParams {
  const float* scale_x;     // [M, kb]
  const float* scale_gate;  // [nb, kb]
  const float* scale_up;    // [nb, kb]
  __nv_bfloat16* out;       // [M, ld_out]
  long long ld_out;
  int m, kb, nb;
  int stages;               // shared-memory ring depth (host: what fits)
  unsigned int* flags;      // [gridDim.x], holds the epoch of the last launch that filled slot i; plus the two
                            // words kStreamSyncLaunches / kStreamSyncTickets below
  float* partials;          // [gridDim.x][2][MPAD][128]
};

// The epoch of a launch is kept on the device, so that a launch recorded once (a CUDA graph) can be replayed: word
// kStreamSyncLaunches of the flag area counts completed launches on this workspace, every CTA reads it when it starts
// and stamps with that count + 1 and takes a ticket (word kStreamSyncTickets) right after reading; the CTA that drew
// the last ticket advances the count when its work is done.  All CTAs have read the count before the last ticket is
// taken.
constexpr int kStreamSyncLaunches = 1022;
constexpr int kStreamSyncTickets = 1023;
static_assert(kStreamMaxGrid <= kStreamSyncLaunches, "hand-off flags and the launch counters share the flag area");

template <int MPAD>
struct StreamCfg {
  static constexpr uint32_t kXTileBytes = MPAD * 128;  // multiple of 1024 for MPAD >= 8
  static constexpr uint32_t kStageBytes = 2 * kOperandTileBytes + kXTileBytes;
  static constexpr uint32_t kTmemCols = kStreamAccStages * 2 * MPAD;  // 128 / 256 / 512
  static constexpr uint32_t kBarBytes = 512;
  __host__ __device__ static constexpr uint32_t smem_bytes(int stages, int kb) {
    return stages * kStageBytes + kBarBytes + static_cast<uint32_t>(kb) * MPAD * 4 + 1024;
  }
};

__device__ __forceinline__ long long stream_range_start(long long units, int ranges, int r) {
  return units * r / ranges;
}

template <int MPAD>
__global__ void __launch_bounds__(kStreamThreads, 1)
gateup_stream_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                     const __grid_constant__ CUtensorMap tm_up, const StreamParams p) {
  using Cfg = StreamCfg<MPAD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t ring = smem_base;
  const uint32_t bars = smem_base + p.stages * Cfg::kStageBytes;
  const uint32_t bar_full = bars;                               // [kStreamMaxStages]
  const uint32_t bar_empty = bars + 8 * kStreamMaxStages;       // [kStreamMaxStages]
  const uint32_t bar_acc_full = bars + 16 * kStreamMaxStages;   // [kStreamAccStages]
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kStreamAccStages;
  const uint32_t tmem_slot = bar_acc_empty + 8 * kStreamAccStages;
  const uint32_t abort_slot = tmem_slot + 4;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_gen = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));
  float* sx_smem = reinterpret_cast<float*>(smem_gen + (bars - smem_base) + Cfg::kBarBytes);  // [kb][MPAD]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Ranges are handed out in reverse block order: a range only ever waits for
  // ranges with a HIGHER index, i.e. blocks with a LOWER blockIdx, which the
  // hardware dispatches first.
  const int ranges = gridDim.x;
  const int my_range = ranges - 1 - static_cast<int>(blockIdx.x);
  const long long units = static_cast<long long>(p.nb) * p.kb;
  const long long u_begin = stream_range_start(units, ranges, my_range);
  const long long u_end = stream_range_start(units, ranges, my_range + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < kStreamAccStages; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 4);  // one arrival per consumer warp
    }
    *abort_gen = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_gate);
    tma_prefetch_desc(&tm_up);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  WaitCtx ctx{abort_slot, false, false};

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      const uint64_t stream_once = l2_policy_evict_first();  // weights are read exactly once
      const uint64_t keep = l2_policy_evict_last();          // the X tiles are re-read by every CTA
      int stage = 0;
      uint32_t phase = 0;
      int nbk = static_cast<int>(u_begin / p.kb);
      int j = static_cast<int>(u_begin - static_cast<long long>(nbk) * p.kb);
      for (long long u = u_begin; u < u_end; ++u) {
        bool ok = mbar_wait(ctx, bar_empty + 8 * stage, phase ^ 1u, kWaitStreamEmpty);
        ok = ok && GU_IN_RANGE(stage >= 0 && stage < p.stages && p.stages <= kStreamMaxStages, kSiteStreamStage) &&
             GU_IN_RANGE(load_coords_ok(p.kb, j, nbk * 128, p.nb * 128), kSiteStreamLoad);
        if (ok) {
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t dst = ring + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(full, Cfg::kStageBytes);
          tma_load_2d_hint(dst, &tm_gate, full, j * kBlockK, nbk * 128, stream_once);
          tma_load_2d_hint(dst + kOperandTileBytes, &tm_up, full, j * kBlockK, nbk * 128, stream_once);
          tma_load_2d_hint(dst + 2 * kOperandTileBytes, &tm_x, full, j * kBlockK, 0, keep);
        }
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        if (++j == p.kb) { j = 0; ++nbk; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------- MMA issuer -------------------------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(128, MPAD);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (long long u = u_begin; u < u_end; ++u) {
        bool ok = mbar_wait(ctx, bar_acc_empty + 8 * acc, acc_phase ^ 1u, kWaitStreamAccEmpty);
        ok = mbar_wait(ctx, bar_full + 8 * stage, phase, kWaitStreamFull) && ok;
        if (ok) {
          tc_fence_after();
          const uint32_t base = ring + stage * Cfg::kStageBytes;
          const uint64_t gdesc = umma_desc_k_sw128(base);
          const uint64_t udesc = umma_desc_k_sw128(base + kOperandTileBytes);
          const uint64_t xdesc = umma_desc_k_sw128(base + 2 * kOperandTileBytes);
          const uint32_t d = tmem_base + acc * (2 * MPAD);
#pragma unroll
          for (int kk = 0; kk < kBlockK / 32; ++kk) {
            umma_f8(d, gdesc + 2 * kk, xdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
            umma_f8(d + MPAD, udesc + 2 * kk, xdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);
          umma_commit(bar_acc_full + 8 * acc);
        }
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        if (++acc == kStreamAccStages) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- consumers --------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // weight row inside the tile = output column inside the block
    const int ctid = threadIdx.x - 64;    // 0..127
    unsigned int epoch = 0;               // this launch's stamp, never 0; only thread ctid == 0 uses it
    unsigned int ticket = 0;              // taken as soon as the count has been read; looked at when the work is done
    if (ctid == 0) {
      epoch = ld_acquire_gpu(p.flags + kStreamSyncLaunches) + 1u;
      if (epoch == 0u) epoch = 1u;
      ticket = atomicAdd(p.flags + kStreamSyncTickets, 1u);
    }
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    // scale_x, transposed to [kb][MPAD] so one K block's token scales are contiguous
    for (int i = ctid; i < p.kb * MPAD; i += 128) {
      const int jj = i / MPAD, t = i - jj * MPAD;
      sx_smem[i] = (t < p.m) ? __ldg(p.scale_x + static_cast<size_t>(t) * p.kb + jj) : 0.f;
    }
    named_bar_sync(1, 128);

    float g[MPAD], up[MPAD];
#pragma unroll
    for (int t = 0; t < MPAD; ++t) { g[t] = 0.f; up[t] = 0.f; }

    int acc = 0;
    uint32_t acc_phase = 0;
    int nbk = static_cast<int>(u_begin / p.kb);
    int j = static_cast<int>(u_begin - static_cast<long long>(nbk) * p.kb);
    int seg_first_j = j;
    float sg_next = 0.f, su_next = 0.f;
    if (GU_IN_RANGE(u_begin >= 0 && u_begin < units && u_end <= units, kSiteStreamScale)) {
      sg_next = __ldg(p.scale_gate + u_begin);  // scale grids are [nb][kb]: unit index == flat index
      su_next = __ldg(p.scale_up + u_begin);
    }

    for (long long u = u_begin; u < u_end; ++u) {
      const float sgw = sg_next, suw = su_next;
      if (u + 1 < u_end) {
        sg_next = __ldg(p.scale_gate + u + 1);
        su_next = __ldg(p.scale_up + u + 1);
      }
      const bool ok = mbar_wait(ctx, bar_acc_full + 8 * acc, acc_phase, kWaitStreamAccFull);
      tc_fence_after();
      {
        constexpr int CH = MPAD < 32 ? MPAD : 32;  // tokens per TMEM read
        const uint32_t t0 = lane_addr + acc * (2 * MPAD);
#pragma unroll
        for (int c = 0; c < MPAD; c += CH) {
          float vg[CH], vu[CH];
          if (ok) {
            if constexpr (CH == 16) {
              tmem_ld16(t0 + c, vg);
              tmem_ld16(t0 + MPAD + c, vu);
            } else {
              tmem_ld32(t0 + c, vg);
              tmem_ld32(t0 + MPAD + c, vu);
            }
            tmem_ld_wait_pin<CH>(vg);
            tmem_ld_wait_pin<CH>(vu);
          } else {
#pragma unroll
            for (int t = 0; t < CH; ++t) { vg[t] = 0.f; vu[t] = 0.f; }
          }
          const float4* sx4 = reinterpret_cast<const float4*>(sx_smem + j * MPAD + c);
#pragma unroll
          for (int t4 = 0; t4 < CH / 4; ++t4) {
            const float4 s = sx4[t4];
            const int t = c + 4 * t4;
            g[t + 0] = fmaf(vg[4 * t4 + 0], s.x * sgw, g[t + 0]);
            g[t + 1] = fmaf(vg[4 * t4 + 1], s.y * sgw, g[t + 1]);
            g[t + 2] = fmaf(vg[4 * t4 + 2], s.z * sgw, g[t + 2]);
            g[t + 3] = fmaf(vg[4 * t4 + 3], s.w * sgw, g[t + 3]);
            up[t + 0] = fmaf(vu[4 * t4 + 0], s.x * suw, up[t + 0]);
            up[t + 1] = fmaf(vu[4 * t4 + 1], s.y * suw, up[t + 1]);
            up[t + 2] = fmaf(vu[4 * t4 + 2], s.z * suw, up[t + 2]);
            up[t + 3] = fmaf(vu[4 * t4 + 3], s.w * suw, up[t + 3]);
          }
        }
      }
      // every read of this TMEM stage has completed: hand it back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
      if (++acc == kStreamAccStages) { acc = 0; acc_phase ^= 1u; }

      const bool block_done = (j == p.kb - 1);
      if (block_done || u + 1 == u_end) {
        // ------------------------- end of a segment -------------------------
        if (seg_first_j != 0) {
          // started mid-block: publish the partial sums for the block's owner
          float* slot = p.partials + static_cast<size_t>(my_range) * (2 * MPAD * 128);
          if (GU_IN_RANGE(my_range >= 0 && my_range < kStreamMaxGrid && row >= 0 && row < 128, kSiteStreamHandOff))
#pragma unroll
          for (int t = 0; t < MPAD; ++t) {
            __stcg(slot + t * 128 + row, g[t]);
            __stcg(slot + (MPAD + t) * 128 + row, up[t]);
          }
          __threadfence();
          named_bar_sync(1, 128);
          if (ctid == 0 && !ctx.aborted) st_release_gpu(p.flags + my_range, epoch);
        } else {
          if (!block_done) {
            // owner of the block's first K block: collect the later ranges' partials, in range order
            const long long block_end = static_cast<long long>(nbk + 1) * p.kb;
            for (int rr = my_range + 1; rr < ranges && stream_range_start(units, ranges, rr) < block_end; ++rr) {
              if (ctid == 0 && !ctx.aborted) {
                unsigned long long t0 = 0;
                for (uint32_t it = 1; ld_acquire_gpu(p.flags + rr) != epoch; ++it) {
                  spin_backoff_ns(64u);
                  if ((it & 255u) == 0u) {
                    const unsigned long long now = globaltimer_ns();
                    if (t0 == 0) {
                      t0 = now;
                    } else if (now - t0 > g_wait_limit_ns || ctx.raised()) {
                      ctx.fail(kWaitStreamFlag, (kWaitStreamFlag << 24) | (blockIdx.x & 0xffffffu));
                      break;
                    }
                  }
                }
              }
              named_bar_sync(1, 128);
              if (!ctx.raised()) {
                const float* slot = p.partials + static_cast<size_t>(rr) * (2 * MPAD * 128);
#pragma unroll
                for (int t = 0; t < MPAD; ++t) {
                  g[t] += __ldcg(slot + t * 128 + row);
                  up[t] += __ldcg(slot + (MPAD + t) * 128 + row);
                }
              }
            }
          }
          // SwiGLU and store: consecutive lanes hold consecutive output columns
          __nv_bfloat16* out_col = p.out + static_cast<size_t>(nbk) * 128 + row;
          if (GU_IN_RANGE(nbk >= 0 && nbk < p.nb && static_cast<long long>(nbk) * 128 + row < p.ld_out, kSiteStreamStore))
#pragma unroll
          for (int t = 0; t < MPAD; ++t) {
            if (t < p.m) out_col[static_cast<size_t>(t) * p.ld_out] = __float2bfloat16_rn(swiglu_bf16(g[t], up[t]));
          }
        }
#pragma unroll
        for (int t = 0; t < MPAD; ++t) { g[t] = 0.f; up[t] = 0.f; }
        seg_first_j = 0;
      }
      if (++j == p.kb) { j = 0; ++nbk; }
    }
    // Whoever drew the launch's last ticket — every CTA had read the count by then — advances the count: the next
    // launch (or a replay of this one) stamps with a new epoch.
    if (ctid == 0 && ticket == gridDim.x - 1u) {
      p.flags[kStreamSyncTickets] = 0u;
      __threadfence();
      atomicAdd(p.flags + kStreamSyncLaunches, 1u);
    }
  }

  // ------------------------------- teardown --------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_gen) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) spin_backoff_ns(1000u);
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace gu
