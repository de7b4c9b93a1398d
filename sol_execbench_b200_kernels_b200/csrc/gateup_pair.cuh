// Persistent tile kernel for CTA pairs: the gate/up projection with fused SwiGLU
// for everything but decode-sized and single-block M.
//
// Two CTAs on neighbouring SMs (a cluster of two) own a 256-token x 128-column
// output tile of BOTH projections.  Each CTA stages its own 128 token rows of X
// and HALF of the weight rows of a K block (the even CTA the gate block, the odd
// CTA the up block: 32 KiB per CTA and K block instead of the 48 KiB a lone CTA
// needs), the even CTA issues one tcgen05.mma stream with cta_group::2 (M = 256,
// N = 256) for both, and each CTA finds the 128 x 256 fp32 partial of its own
// tokens in its own TMEM: gate in columns [0,128), up in [128,256) of a
// two-stage accumulator.  Per MAC that is two thirds of the shared-memory traffic
// (TMA writes and MMA operand reads) of the lone-CTA kernel.
//
// What bounds a kernel of this kind is the round trip of an accumulator stage —
// MMA, completion seen by the consumers, the partial read out of TMEM, the stage
// handed back, the next MMA issued — because the fp32 per-128 scales force every
// K block's partial through registers and TMEM holds only two 128 x 256 stages.
// So every hop of that loop is kept short:
//   * the issuer and the producer are whole warps in uniform control flow with one
//     elected lane doing the work (descriptors and addresses stay in uniform
//     registers), and the polls a step needs are issued together;
//   * exactly one lane per warp polls a barrier (the other 31 wait at a warp or
//     CTA barrier), so polling does not load the shared-memory pipeline that the
//     barriers themselves go through;
//   * arrivals that cross to the other CTA are relaxed (what they order lives in
//     TMEM) and one commit per CTA and K block serves both the ring slot and the
//     accumulator;
//   * warps 4-7 promote the gate half and warps 8-11 the up half (a thread owns
//     one token row and all 128 columns of one projection), reading the partial
//     in pieces through two alternating buffers so that the tcgen05.ld of a
//     piece is in flight while the piece before it is multiplied by
//     scale_x[m, kb] * scale_w[n/128, kb] and added to the fp32 running sums
//     (block order ascending, as the reference's promotion loop does:
//     variants/cute_fused_v1/blockwise_gemm_fused.py:1817-1823); the stage goes
//     back as soon as the last piece is in registers;
//   * at the end of a tile the consumers only round gate and up to bf16 into a
//     64 KiB shared-memory hand-over tile and go on with the next tile; separate
//     epilogue warps apply SiLU, the product and the last rounding in place and
//     issue the TMA store.
//
// Warp roles:
//   warp 0        TMA producer: own X tile + own 128 weight rows (gate or up)
//   warp 1        TMEM allocation; in the even CTA it issues every MMA of the pair
//   warps 4-11    consumers (promotion); warp w reads TMEM lanes 32*(w%4)..+31
//   epilogue      warps 2-3 (12 warps per CTA, the default) or warps 12-15 (16)
//
// Cross-CTA signalling: every wait is on a barrier of the waiting CTA and is
// bounded; the other CTA reaches it with shared::cluster addresses (remote
// mbarrier.arrive, TMA completion bytes, tcgen05.commit).  No multicast form.
#pragma once

#include "gateup_tile.cuh"

namespace gu {

#ifndef GU_PAIR_THREADS
#define GU_PAIR_THREADS 384
#endif
#ifndef GU_PIECE
#define GU_PIECE 16
#endif
#ifndef GU_INFLIGHT
#define GU_INFLIGHT 2
#endif
constexpr int kPairThreads = GU_PAIR_THREADS;                    // 384: epilogue on warps 2-3; 512: on warps 12-15
constexpr int kPairEpiWarp0 = kPairThreads == 512 ? 12 : 2;
constexpr int kPairEpiThreads = kPairThreads == 512 ? 128 : 64;
constexpr int kPairConsumerRegs = kPairThreads == 512 ? 216 : 232;  // the other warpgroups keep 40
#ifndef GU_PAIR_STAGES
#define GU_PAIR_STAGES 4
#endif
constexpr int kPairStages = GU_PAIR_STAGES;                      // shared-memory ring depth
constexpr uint32_t kPairStageBytes = 2 * kOperandTileBytes;      // X tile + this CTA's half of the weight rows
constexpr uint32_t kPairHandBytes = 4 * kTileOutHalfBytes;       // bf16 gate tile + bf16 up tile (two half tiles each)
constexpr uint32_t kPairSmemBytes = kPairStages * kPairStageBytes + kPairHandBytes + 256 /*barriers*/ + 1024 /*alignment*/;
constexpr int kPairPiece = GU_PIECE;                             // accumulator columns per tcgen05.ld of a consumer
constexpr int kPairInFlight = GU_INFLIGHT;                       // loads a consumer keeps in flight (1 or 2)
constexpr int kPairRounds = kTileN / (kPairPiece * kPairInFlight);  // rounds of loads per 128-column half

enum : unsigned {
  kWaitPairSlot = 11, kWaitPairFull = 12, kWaitPairStageFree = 13, kWaitPairDone = 14,
  kWaitPairHandEmpty = 15, kWaitPairHandFull = 16, kWaitPairFlag = 17,
};

// Study builds (never the shipped library; see build.py):
//   -DGU_TRACE   per-role cycle counters and time stamps of the first CTA pair, read with gu_trace_read
//   -DGU_EXP=n   results are wrong on purpose; what is left bounds a part of the kernel from above:
//                1 consumers read the partial but skip the promotion arithmetic
//                2 consumers neither read nor add: only the hand-shake with the issuer is left
//                3 the issuer waits for each K block's completion before going on (issue-to-completion latency)
//                4 as 2, and the issuer never waits for the consumers: MMA + TMA + issuer alone
//                5 as 3 and 4 together: one K block in flight on an otherwise idle SM
//                6 consumers do the promotion arithmetic on stale registers but never read TMEM
//                7 consumers read only 64 of their 128 columns (two rounds of loads) before the stage goes back, all
//                  the arithmetic still done; 8 as 7 with the arithmetic of those 64 columns only
//               10 consumers read 64 columns in one batch, hand the stage back at once, then do all the arithmetic
//                9 the epilogue warps skip the SwiGLU arithmetic (what their instruction stream costs the consumer
//                  warps that share their schedulers)
//   -DGU_PAIR_THREADS=512, -DGU_PIECE=32, -DGU_INFLIGHT=1, -DGU_PAIR_STAGES=5, -DGU_CONSUMER_ROUNDS   layout variants that were measured
//   -DGU_ISSUER2 two issuing threads in the even CTA (warps 0 and 1 each fill the ring slots and issue the K blocks of
//                one parity); results are right, 3.6 % slower than one issuer (0.437 against 0.422 ms at 4096 tokens)
#ifdef GU_TRACE
// Cycle counters of cluster 0 (both CTAs), summed over the launch: [rank][slot]
//  0 producer: waiting for a free ring slot     1 issuer: waiting for operands   2 issuer: waiting for a free unit
//  3 consumer warp 4: waiting for a partial     4 consumer warp 4: in tcgen05.wait::ld
//  5 consumer warp 4: K loop, all tiles         6 consumer warp 4: hand-over (incl. waiting for the tile to be free)
//  7 first epilogue warp: SwiGLU + store       8 first epilogue warp: waiting for a hand-over
//  9 whole CTA (thread 0)                      10 K blocks walked by consumer warp 4
__device__ unsigned long long g_trace[2][16];
// Time stamps (clock64 of the CTA's SM) of K blocks 8..23 of cluster 0's first tile, four per K block: [rank][role][64]
//  role 0, issuer (even CTA): operands and stage seen / - / MMAs issued / commits issued
//  role 1, consumer warp 4:   partial seen / - / last load issued / stage handed back
__device__ unsigned long long g_events[2][2][64];
#define GU_EV(role, j, e) do { if (tr_me && tr_first && (j) >= 8 && (j) < 24) g_events[blockIdx.x & 1][role][4 * ((j) - 8) + (e)] = clock64(); } while (0)
// one reporting thread per role: the elected lane of the producer and issuer warps, lane 0 of consumer warp 4 and of the
// first epilogue warp
#define GU_TR_DECL                                                                                               \
  unsigned long long tr_t0 = 0;                                                                                  \
  bool tr_me = blockIdx.x < 2 && (threadIdx.x == 128 || threadIdx.x == 32 * kPairEpiWarp0)
#define GU_TR_BEGIN() do { if (tr_me) tr_t0 = clock64(); } while (0)
// (reductions whose result is not used: the thread does not wait for them)
#define GU_TR_END(slot) do { if (tr_me) atomicAdd(&g_trace[blockIdx.x & 1][slot], (unsigned long long)(clock64() - tr_t0)); } while (0)
#else
#define GU_TR_DECL
#define GU_TR_BEGIN() do {} while (0)
#define GU_TR_END(slot) do {} while (0)
#define GU_EV(role, j, e) do {} while (0)
#endif


// packed FMAs over one piece: sums[i] += piece[2i, 2i+1] * scale
__device__ __forceinline__ void pair_fma(float2* sums, const float* piece, float2 scale) {
#if defined(GU_EXP) && (GU_EXP == 1 || GU_EXP == 2 || GU_EXP == 4 || GU_EXP == 5)
  sums[0].x += piece[0] * scale.x;  // experiment: no promotion arithmetic
  return;
#endif
#pragma unroll
  for (int i = 0; i < kPairPiece / 2; ++i)
    sums[i] = __ffma2_rn(make_float2(piece[2 * i], piece[2 * i + 1]), scale, sums[i]);
}

__device__ __forceinline__ void pair_ld(uint32_t taddr, float* v) {
#if defined(GU_EXP) && (GU_EXP == 2 || GU_EXP == 4 || GU_EXP == 5 || GU_EXP == 6)
  (void)taddr;  // experiment: the partial is not read at all
  (void)v;
#else
  if constexpr (kPairPiece == 32) tmem_ld32(taddr, v);
  else tmem_ld16(taddr, v);
#endif
}

// One lane of a converged warp polls; every lane gets the outcome.  Keeps the warp's control flow uniform (so the
// addresses and descriptors around it stay in uniform registers) and the polling traffic at one thread per warp.
__device__ __forceinline__ bool mbar_wait_elected(WaitCtx& ctx, bool elected, uint32_t bar, uint32_t parity, unsigned code) {
  bool ok = true;
  if (elected) ok = mbar_wait(ctx, bar, parity, code);
  ok = __all_sync(0xffffffffu, ok);
  __syncwarp();  // what the polling lane acquired is ordered before the other lanes' accesses
  return ok;
}
// Same for waiters that do not branch on the outcome (after a time-out they read stale data, which is discarded).
__device__ __forceinline__ void mbar_wait_lane(WaitCtx& ctx, bool elected, uint32_t bar, uint32_t parity, unsigned code) {
  if (elected) (void)mbar_wait(ctx, bar, parity, code);
  __syncwarp();
}

// TileParams as used here: num_m_blocks / group_m count 256-token pair blocks, num_tiles pair tiles.
//
// kSingle: the same pipeline as a plain block-scaled GEMM, C = bf16(sum_kb scale_a * scale_b * (A_kb . B_kb^T)) — the
// GEMM the reference launches twice (kernel.py:487-488); here the MLP's down projection.  The two 128-row weight
// tiles of a K block are then two ADJACENT 128-column blocks of one B matrix (tm_gate; scale rows 2n and 2n+1 of
// scale_gate), a pair tile is 256 x 256 outputs, and the epilogue warps only issue the stores of the handed-over tiles.
//
// kStreamK: the launch's first TileParams::tile_begin tiles (a whole number of rounds) are dealt out round-robin as
// whole tiles, as without it; the (tile, K block) units of the remaining tiles — between one and two rounds' worth —
// are cut into one contiguous range per cluster, all ranges equal to within one unit, so that no cluster idles
// through a last partial round of tiles.  A range starts in the middle of a tile at most once (its first segment) and
// ends in the middle of one at most once (its last segment).  The cluster that holds a tile's FIRST K blocks owns the
// tile: the cluster after it, which begins with the tile's remaining K blocks, writes the running sums of that
// remainder to its slot of a scratch array and stamps its flag with the launch's epoch; the owner, which reaches the
// tile at the very end of its own range, finds the flag stamped, adds the remainder (ascending block order inside
// both parts, one fp32 addition joining them) and hands the tile to its epilogue warps as usual.  Only the host picks
// this schedule, and only when the launch has at least as many tiles as clusters (so a tile spans at most two
// ranges).  (Cutting ALL units into contiguous ranges was measured too: the clusters then walk different weight
// blocks at any moment and the launch loses more in L2 misses than it gains: 491 against 441 us on 4096 tokens.)
// The epoch lives on the device (a count of launches in the scratch area, read by every CTA at its start and
// advanced by the last CTA to have read it), so a recorded launch can be replayed.
constexpr int kPairFlagWord0 = 512;        // words [512, 512 + CTAs) of the flag area: hand-off stamps, one per CTA
constexpr int kPairSyncLaunches = 1020;    // finished launches on this scratch area
constexpr int kPairSyncTickets = 1021;     // CTAs of the running launch that have left
constexpr int kPairMaxCtas = 448;          // 1020 - 512, rounded down to a pair count with room to spare

template <bool kStreamK>
struct PairWalk {
  long long u, u_end;  // stream-K: this cluster's unit range
  int cur, step;       // data-parallel: next tile, clusters
  __device__ __forceinline__ PairWalk(const TileParams& p, int cluster_id, int clusters) {
    if constexpr (kStreamK) {
      const long long units = static_cast<long long>(p.num_tiles - p.tile_begin) * p.kb;
      u = units * cluster_id / clusters;
      u_end = units * (cluster_id + 1) / clusters;
      cur = cluster_id;
      step = clusters;
    } else {
      u = u_end = 0;
      cur = cluster_id;
      step = clusters;
    }
  }
  // no segment is left
  __device__ __forceinline__ bool done(const TileParams& p) const {
    if constexpr (kStreamK) return cur >= p.tile_begin && u >= u_end;
    else return cur >= p.num_tiles;
  }
  // next segment: K blocks [jb, je) of `tile`
  __device__ __forceinline__ bool next(const TileParams& p, int& tile, int& jb, int& je) {
    if constexpr (kStreamK) {
      if (cur < p.tile_begin) {  // the whole rounds first
        tile = cur;
        cur += step;
        jb = 0;
        je = p.kb;
        return true;
      }
      if (u >= u_end) return false;
      const int rel = static_cast<int>(u / p.kb);
      tile = p.tile_begin + rel;
      jb = static_cast<int>(u - static_cast<long long>(rel) * p.kb);
      const long long seg_end = min(static_cast<long long>(rel + 1) * p.kb, u_end);
      je = jb + static_cast<int>(seg_end - u);
      u = seg_end;
      return true;
    } else {
      if (cur >= p.num_tiles) return false;
      tile = cur;
      cur += step;
      jb = 0;
      je = p.kb;
      return true;
    }
  }
};

//
// kMode selects what the epilogue warps do with a finished tile:
//   kPairPlain    SwiGLU (or, kSingle, nothing) and the TMA stores into outs[0]
//   kPairGather   SwiGLU, then the tile is stored into every rank's buffer at this rank's column offset (own and
//                 peers' over NVLink; plain TMA stores, no load touches peer memory): the all-gather of a
//                 column-sharded result inside the epilogue (TileParams::out_count, out_rank, out_col0)
//   kPairScatter  kSingle only: the tile of a row-parallel GEMM's partial result goes to the rank that owns its
//                 token block, into the sending rank's slot (TileParams::blocks_per_owner, slot_rows)
//   kPairFp8Out   SwiGLU, then the tile is re-quantised to e4m3 with one fp32 scale per token and 128 columns
//                 (amax / 448; the tile is exactly one scale block wide) and stored as e4m3 + scales: the operand
//                 format of the next block-scaled GEMM.  Bits equal quantising the bf16 result.
enum : int { kPairPlain = 0, kPairGather = 1, kPairScatter = 2, kPairFp8Out = 3 };

// |a|, |b| of a packed bf16 pair folded into a running maximum
__device__ __forceinline__ float amax_bf16x2(float m, uint32_t pr) {
  return fmaxf(m, fmaxf(fabsf(__uint_as_float(pr << 16)), fabsf(__uint_as_float(pr & 0xffff0000u))));
}
// four e4m3 from two packed bf16 pairs: v / sc correctly rounded (reciprocal, then one exact-residual step), then
// round-to-nearest-even with saturation
__device__ __forceinline__ uint32_t e4m3x4_from_bf16x4(uint32_t p0, uint32_t p1, float sc, float rc) {
  uint32_t word = 0;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t pr = e ? p1 : p0;
    const float a = __uint_as_float(pr << 16), b = __uint_as_float(pr & 0xffff0000u);
    const float qa0 = a * rc, qb0 = b * rc;
    const float qa = fmaf(fmaf(-qa0, sc, a), rc, qa0), qb = fmaf(fmaf(-qb0, sc, b), rc, qb0);
    word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qa, qb), __NV_SATFINITE, __NV_E4M3)) << (16 * e);
  }
  // (the residual step turns a quotient of -0 into +0; the sources' sign bits — the high byte of each bf16, gathered by
  // one byte permute — put the sign of such a zero back; a quotient never has the other sign)
  return word | (__byte_perm(p0, p1, 0x7531) & 0x80808080u);
}

// SiLU(gate) * up with the three roundings, in place over the handed-over tiles: 16-byte chunk q of the gate tile
// meets chunk q of the up tile (same layout); chunks first, first + stride, ... of the 2048 belong to this thread
__device__ __forceinline__ void pair_swiglu_chunks(uint8_t* hand_gen, int first, int stride) {
#pragma unroll 4
  for (int q = first; q < 2048; q += stride) {
    uint4* gq = reinterpret_cast<uint4*>(hand_gen + q * 16);
    const uint4 a = *gq;
    const uint4 b = *reinterpret_cast<const uint4*>(hand_gen + 2 * kTileOutHalfBytes + q * 16);
    uint4 o;
    o.x = swiglu_packed_bf16x2(a.x, b.x);
    o.y = swiglu_packed_bf16x2(a.y, b.y);
    o.z = swiglu_packed_bf16x2(a.z, b.z);
    o.w = swiglu_packed_bf16x2(a.w, b.w);
    *gq = o;
  }
}
// The SwiGLU of a cluster's LAST tile has nothing to hide behind (4 - 5 us on two warps: two special-function
// operations per output), so the eight consumer warps, idle by then, share it with the epilogue warps: 2 us per
// launch.  (Not in the stream-K kernel: with this code in it the same K loop measured 165 cycles per block slower,
// 78.0 against 75.8 us at 512 x 4096 x 14336, for a reason that -Xptxas -v does not show.)
constexpr int kPairAllHands = kPairEpiThreads + 256;
#ifdef GU_ISSUER2
// study: in the even CTA warps 0 and 1 each fill the ring slots of one parity and issue the K blocks of that parity
constexpr bool kPairTwoIssuers = true;
#else
constexpr bool kPairTwoIssuers = false;
#endif

template <bool kSingle, int kMode = kPairPlain, bool kStreamK = false>
__device__ __forceinline__ void pair_kernel_body(const CUtensorMap& tm_x, const CUtensorMap& tm_gate,
                                                 const CUtensorMap& tm_up, const CUtensorMap* outs,
                                                 const TileParams& p) {
#ifdef GU_NO_SHARED_EPILOGUE  // study build: the last tile's SwiGLU stays on the epilogue warps
  constexpr bool kShareLast = false;
#else
  constexpr bool kShareLast = !kSingle && kMode != kPairFp8Out && !kStreamK;
#endif
  static_assert(kMode != kPairScatter || kSingle, "scatter is a mode of the plain GEMM");
  static_assert((kMode != kPairGather && kMode != kPairFp8Out) || !kSingle, "gather / fp8 output are modes of gate/up");
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern; both CTAs of a pair get the same offsets
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t ring = smem_base;
  const uint32_t hand = smem_base + kPairStages * kPairStageBytes;  // gate tile (later the output tile), then up tile
  const uint32_t bars = hand + kPairHandBytes;
  const uint32_t bar_full = bars;                           // [stages] even CTA's are used: 2 producer arrivals + both CTAs' bytes
  const uint32_t bar_done = bar_full + 8 * kPairStages;     // [stages] the K block's MMAs have completed (one commit):
                                                            // its partial is in TMEM and its ring slot may be refilled
  const uint32_t bar_stage_free = bar_done + 8 * kPairStages;  // [2] even CTA's are used: 8 consumer warps x 2 CTAs
  const uint32_t bar_hand_full = bar_stage_free + 16;       // 8 consumer warps
  const uint32_t bar_hand_empty = bar_hand_full + 8;        // the storing epilogue thread
  const uint32_t tmem_slot = bar_hand_empty + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_gen = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));
  volatile unsigned int* epoch_gen = reinterpret_cast<volatile unsigned int*>(smem_gen + (abort_slot + 4 - smem_base));

  // the warp index through a shuffle, so that the compiler knows it is the same in every lane
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the MMAs
  const int cluster_id = blockIdx.x >> 1;
  const int clusters = gridDim.x >> 1;
  GU_TR_DECL;
#ifdef GU_TRACE
  const unsigned long long tr_cta0 = clock64();
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);
      mbar_init(bar_done + 8 * s, 1);
    }
    for (int q = 0; q < 2; ++q) mbar_init(bar_stage_free + 8 * q, 16);
    mbar_init(bar_hand_full, 8);
    mbar_init(bar_hand_empty, 1);
    *abort_gen = 0;
    *epoch_gen = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_gate);
    tma_prefetch_desc(&tm_up);
    if constexpr (kMode == kPairGather || kMode == kPairScatter) {
      for (int r = 0; r < p.out_count; ++r) tma_prefetch_desc(&outs[r]);
    } else {
      tma_prefetch_desc(&outs[0]);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTileTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers and the abort flag of both CTAs exist before anything reaches across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  WaitCtx ctx{abort_slot, false, true};
  const bool is_consumer = warp >= 4 && warp < 12;
  const bool is_epilogue = warp >= kPairEpiWarp0 && warp < kPairEpiWarp0 + kPairEpiThreads / 32;

  if (!is_consumer) {
    reg_dealloc<40>();
    if (warp == 0 || (kPairTwoIssuers && warp == 1 && rank == 0)) {
      // ---------------- TMA producer: the whole warp walks the loop, one elected lane waits and issues ----------------
      const bool elected = elect_one() != 0u;
      // (two issuers) parity of the slots and K blocks this warp owns; -1: every slot, no block
      const int own = (kPairTwoIssuers && rank == 0) ? (warp == 0 ? 1 : 0) : -1;
      uint32_t next_issue = own < 0 ? 0u : static_cast<uint32_t>(own);
      const uint32_t tmem_u2 = kPairTwoIssuers ? __shfl_sync(0xffffffffu, tmem_base, 0) : 0u;
      const uint32_t done_odd2 = kPairTwoIssuers ? mapa_shared(bar_done, 1) : 0u;
      auto issue_own = [&](uint32_t b) {
        constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * kTileM, 2 * kTileN);
        const uint32_t stage = b % kPairStages, phase = (b / kPairStages) & 1u;
        const uint32_t acc = b & 1u, acc_phase = (b >> 1) & 1u;
        const uint64_t adesc = umma_desc_k_sw128(ring) + stage * (kPairStageBytes >> 4);
        const uint64_t bdesc = umma_desc_k_sw128(ring + kOperandTileBytes) + stage * (kPairStageBytes >> 4);
        const uint32_t d = tmem_u2 + acc * (2 * kTileN);
        bool ok = true;
        if (elected) {
          const uint32_t hit_full = mbar_try_wait(bar_full + 8 * stage, phase);
          const uint32_t hit_free = mbar_try_wait(bar_stage_free + 8 * acc, acc_phase ^ 1u);
          ok = hit_full || mbar_wait(ctx, bar_full + 8 * stage, phase, kWaitPairFull);
          ok = (hit_free || mbar_wait(ctx, bar_stage_free + 8 * acc, acc_phase ^ 1u, kWaitPairStageFree)) && ok;
        }
        if (ok && elected) {
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kBlockK / 32; ++kk)
            umma_f8_pair(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          umma_commit_pair(bar_done + 8 * stage);
          umma_commit_pair(done_odd2 + 8 * stage);
        }
        __syncwarp();
      };
#ifdef GU_TRACE
      tr_me = blockIdx.x < 2 && elected;
#endif
      const uint32_t full_even = mapa_shared(bar_full, 0);
      uint32_t slots = 0;  // ring slots filled so far: stage = low bits, barrier phase = the next bit
      PairWalk<kStreamK> walk(p, cluster_id, clusters);
      int tile, jb, je;
      while (walk.next(p, tile, jb, je)) {
        int pm, nb;
        tile_coords(p, tile, pm, nb);
        const int row0 = (2 * pm + static_cast<int>(rank)) * kTileM;
        for (int j = jb; j < je; ++j, ++slots) {
          const uint32_t stage = slots % kPairStages, phase = (slots / kPairStages) & 1u;
          if (kPairTwoIssuers && own >= 0 && static_cast<int>(slots & 1u) != own) continue;
          GU_TR_BEGIN();
          const bool ok = mbar_wait_elected(ctx, elected, bar_done + 8 * stage, phase ^ 1u, kWaitPairSlot);
          GU_TR_END(0);
          const uint32_t full = full_even + 8 * stage;
          const uint32_t dst = ring + stage * kPairStageBytes;
          const int b_row = kSingle ? (2 * nb + static_cast<int>(rank)) * kTileN : nb * kTileN;
          (void)b_row;  // (only the range-checked build looks at it)
          if (ok && elected && GU_IN_RANGE(stage < kPairStages, kSitePairStage) &&
              GU_IN_RANGE(load_coords_ok(p.kb, j, row0, 2 * p.num_m_blocks * kTileM) &&
                              load_coords_ok(p.kb, j, b_row, (kSingle ? 2 : 1) * p.num_n_blocks * kTileN), kSitePairLoad)) {
            mbar_arrive_expect_tx_cluster(full, kPairStageBytes);
            tma_load_2d_pair(dst, &tm_x, full, j * kBlockK, row0);  // rows past M read as zero
            if constexpr (kSingle) {
              // B rows [0, 128) of the MMA = column block 2 nb of the one B matrix (even CTA), [128, 256) = block
              // 2 nb + 1 (odd CTA; rows past N read as zero)
              tma_load_2d_pair(dst + kOperandTileBytes, &tm_gate, full, j * kBlockK,
                               (2 * nb + static_cast<int>(rank)) * kTileN);
            } else {
              // B rows [0, 128) of the MMA = the gate block (even CTA), [128, 256) = the up block (odd CTA)
              tma_load_2d_pair(dst + kOperandTileBytes, rank == 0 ? &tm_gate : &tm_up, full, j * kBlockK, nb * kTileN);
            }
          }
          __syncwarp();
          if constexpr (kPairTwoIssuers) {
            if (own >= 0) {
              for (; next_issue + 2 <= slots; next_issue += 2) issue_own(next_issue);
            }
          }
        }
      }
      if constexpr (kPairTwoIssuers) {
        if (own >= 0) {
          for (; next_issue < slots; next_issue += 2) issue_own(next_issue);
          // the odd CTA's last hand-backs must have landed here before this CTA may go away
          for (uint32_t b = slots; b < slots + 2; ++b)
            mbar_wait_elected(ctx, elected, bar_stage_free + 8 * (b & 1u), ((b >> 1) & 1u) ^ 1u, kWaitPairStageFree);
        }
      }
      // the last commits into this CTA's ring barriers must have landed before the CTA may go away
      for (int s = 0; s < kPairStages; ++s, ++slots)
        mbar_wait_elected(ctx, elected, bar_done + 8 * (slots % kPairStages), ((slots / kPairStages) & 1u) ^ 1u,
                          kWaitPairSlot);
    } else if (!kPairTwoIssuers && warp == 1 && rank == 0) {
      // ---------------- MMA issuer of the pair: the whole warp walks the loop, one elected lane waits and issues ------
      const bool elected = elect_one() != 0u;
#ifdef GU_TRACE
      tr_me = blockIdx.x < 2 && elected;
#endif
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * kTileM, 2 * kTileN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t done_odd = mapa_shared(bar_done, 1);
      // descriptors of ring stage 0; a stage further on adds its byte offset >> 4 to the address field (low word)
      const uint64_t adesc0 = umma_desc_k_sw128(ring);
      const uint64_t bdesc0 = umma_desc_k_sw128(ring + kOperandTileBytes);
      uint32_t blocks = 0;  // K blocks issued so far
      PairWalk<kStreamK> walk(p, cluster_id, clusters);
      int tile, jb, je;
#ifdef GU_TRACE
      bool tr_first = true, tr_seen = false;
#endif
      while (walk.next(p, tile, jb, je)) {
#ifdef GU_TRACE
        tr_first = !tr_seen;
        tr_seen = true;
#endif
        for (int j = jb; j < je; ++j, ++blocks) {
          const uint32_t stage = blocks % kPairStages, phase = (blocks / kPairStages) & 1u;
          const uint32_t acc = blocks & 1u, acc_phase = (blocks >> 1) & 1u;
          const uint64_t adesc = adesc0 + stage * (kPairStageBytes >> 4);
          const uint64_t bdesc = bdesc0 + stage * (kPairStageBytes >> 4);
          const uint32_t d = tmem_u + acc * (2 * kTileN);
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t stage_free = bar_stage_free + 8 * acc;
          // The two polls are issued back to back (a poll of shared memory takes a hundred cycles or more while TMA
          // writes and MMA operand reads keep it busy); only a poll that fails turns into a wait.
          bool ok = true;
          GU_TR_BEGIN();
          if (elected) {
            const uint32_t hit_full = mbar_try_wait(full, phase);
            const uint32_t hit_free = mbar_try_wait(stage_free, acc_phase ^ 1u);
            ok = hit_full || mbar_wait(ctx, full, phase, kWaitPairFull);
#if !(defined(GU_EXP) && (GU_EXP == 4 || GU_EXP == 5))  // (experiments 4, 5: the issuer never waits for the consumers)
            ok = (hit_free || mbar_wait(ctx, stage_free, acc_phase ^ 1u, kWaitPairStageFree)) && ok;
#endif
          }
          // (only the elected lane looks at `ok`; the others walk the loop whatever it is, so no vote is needed between
          // the wake-up and the first MMA)
          GU_TR_END(1);
          GU_EV(0, j, 0);
          if (ok && elected) {
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kBlockK / 32; ++kk)  // 32 e4m3 along K inside the swizzle span: +2 in the address field
              umma_f8_pair(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
            GU_EV(0, j, 2);
            umma_commit_pair(bar_done + 8 * stage);  // to both CTAs: partial in TMEM, operands read
            umma_commit_pair(done_odd + 8 * stage);
            GU_EV(0, j, 3);
#if defined(GU_EXP) && (GU_EXP == 3 || GU_EXP == 5)
            mbar_wait(ctx, bar_done + 8 * stage, phase, kWaitPairDone);  // experiment: issue-to-completion latency
            GU_EV(0, j, 1);
#endif
          }
          __syncwarp();
        }
      }
      // the odd CTA's last hand-backs must have landed here before this CTA may go away
      for (uint32_t b = blocks; b < blocks + 2; ++b)
        mbar_wait_elected(ctx, elected, bar_stage_free + 8 * (b & 1u), ((b >> 1) & 1u) ^ 1u, kWaitPairStageFree);
    } else if (is_epilogue) {
      // -------------------------------- epilogue ---------------------------------
      const int et = static_cast<int>(threadIdx.x) - 32 * kPairEpiWarp0;  // 0 .. kPairEpiThreads-1
      uint8_t* hand_gen = smem_gen + (hand - smem_base);
      uint32_t hand_phase = 0;
      if constexpr (kStreamK) {
        if (et == 0) {
          // This launch's stamp: launches counted on the scratch area + 1, never 0 (done here, off the other roles'
          // way: they need it a tile part later at the earliest).  The CTA takes its ticket as soon as it has read
          // the count; the last ticket of the launch advances the count for the next launch (or a replay of this
          // one) — by then every CTA of this launch holds its stamp, and launches that share a scratch area never
          // overlap.
          unsigned int e = ld_acquire_gpu(p.flags + kPairSyncLaunches) + 1u;
          if (e == 0u) e = 1u;
          *epoch_gen = e;
          if (atomicAdd(p.flags + kPairSyncTickets, 1u) == gridDim.x - 1u) {
            p.flags[kPairSyncTickets] = 0u;
            __threadfence();
            atomicAdd(p.flags + kPairSyncLaunches, 1u);
          }
        }
      }
      PairWalk<kStreamK> walk(p, cluster_id, clusters);
      int tile, jb, je;
      while (walk.next(p, tile, jb, je)) {
        if (jb != 0) continue;  // (stream-K) the remainder of a tile another cluster owns: nothing is handed over
        // (a cluster's last segment is always the head or the whole of a tile it owns)
        const bool last_tile = kShareLast && walk.done(p);
        int pm, nb;
        tile_coords(p, tile, pm, nb);
        const int row0 = (2 * pm + static_cast<int>(rank)) * kTileM;
        GU_TR_BEGIN();
        // one thread polls; the others sleep at a hardware barrier instead of polling shared memory for a whole tile
        bool ok = true;
        if (et == 0) ok = mbar_wait(ctx, bar_hand_full, hand_phase, kWaitPairHandFull);
        named_bar_sync(2, kPairEpiThreads);
        GU_TR_END(8);
        GU_TR_BEGIN();
        if constexpr (kSingle) {
          // both handed-over tiles are final (and fenced by their writers): four half-tile stores, nothing to compute
          if (et == 0) {
            if (ok && !ctx.aborted && row0 < p.m &&
                GU_IN_RANGE(p.out_cols == 0 || (2 * nb * kTileN + 128 <= p.out_cols && row0 >= 0 && row0 < p.out_rows),
                            kSitePairStore)) {
              const CUtensorMap* dst = &outs[0];
              int y = row0;
              if constexpr (kMode == kPairScatter) {
                // partial result of a row-parallel GEMM: plain TMA store into the owner rank's buffer (over NVLink
                // unless it is this rank), in the slot reserved for this rank; the owner sums the slots
                const int mb = 2 * pm + static_cast<int>(rank);  // this CTA's 128-token block
                const int owner = mb / p.blocks_per_owner;
                y = p.out_rank * p.slot_rows + (mb - owner * p.blocks_per_owner) * kTileM;
                dst = &outs[owner];
              }
              tma_store_2d(dst, hand, 2 * nb * kTileN, y);
              tma_store_2d(dst, hand + kTileOutHalfBytes, 2 * nb * kTileN + 64, y);
              if (2 * nb + 1 < p.n_blocks128) {
                tma_store_2d(dst, hand + 2 * kTileOutHalfBytes, (2 * nb + 1) * kTileN, y);
                tma_store_2d(dst, hand + 3 * kTileOutHalfBytes, (2 * nb + 1) * kTileN + 64, y);
              }
              tma_store_commit();
              tma_store_wait_read0();
            }
            mbar_arrive(bar_hand_empty);
          }
        } else if constexpr (kMode == kPairFp8Out) {
          // A thread owns whole rows (et, et + 64, ...): SwiGLU in place over the row's 16 chunks with the row's
          // largest magnitude, then the row's 128 e4m3 into the bytes the row's first 64 up values occupied (this
          // thread has read them all), in the staging layout of a 128-byte-row tile.
#pragma unroll 1
          for (int r = et; r < kTileM; r += kPairEpiThreads) {
            uint8_t* grow = hand_gen + r * 128;
            uint8_t* urow = grow + 2 * kTileOutHalfBytes;
            float amax = 0.f;
#pragma unroll 4
            for (int c = 0; c < 16; ++c) {
              const uint32_t off = (c >> 3) * kTileOutHalfBytes + (((c & 7) ^ (r & 7)) << 4);
              const uint4 a = *reinterpret_cast<const uint4*>(grow + off);
              const uint4 b = *reinterpret_cast<const uint4*>(urow + off);
              uint4 o;
              o.x = swiglu_packed_bf16x2(a.x, b.x);
              o.y = swiglu_packed_bf16x2(a.y, b.y);
              o.z = swiglu_packed_bf16x2(a.z, b.z);
              o.w = swiglu_packed_bf16x2(a.w, b.w);
              amax = amax_bf16x2(amax_bf16x2(amax_bf16x2(amax_bf16x2(amax, o.x), o.y), o.z), o.w);
              *reinterpret_cast<uint4*>(grow + off) = o;
            }
            const float sc = fmaxf(amax, 1e-12f) / 448.0f;
            const float rc = __frcp_rn(sc);
#pragma unroll 2
            for (int q = 0; q < 8; ++q) {  // 8 chunks of 16 e4m3, each from two chunks of 8 bf16
              const uint32_t off0 = ((2 * q) >> 3) * kTileOutHalfBytes + ((((2 * q) & 7) ^ (r & 7)) << 4);
              const uint32_t off1 = ((2 * q + 1) >> 3) * kTileOutHalfBytes + ((((2 * q + 1) & 7) ^ (r & 7)) << 4);
              const uint4 o0 = *reinterpret_cast<const uint4*>(grow + off0);
              const uint4 o1 = *reinterpret_cast<const uint4*>(grow + off1);
              uint4 w;
              w.x = e4m3x4_from_bf16x4(o0.x, o0.y, sc, rc);
              w.y = e4m3x4_from_bf16x4(o0.z, o0.w, sc, rc);
              w.z = e4m3x4_from_bf16x4(o1.x, o1.y, sc, rc);
              w.w = e4m3x4_from_bf16x4(o1.z, o1.w, sc, rc);
              *reinterpret_cast<uint4*>(urow + ((q ^ (r & 7)) << 4)) = w;
            }
            if (row0 + r < p.m && GU_IN_RANGE(nb >= 0 && nb < p.n_blocks128, kSitePairScaleOut))
              p.scale_out[static_cast<size_t>(row0 + r) * p.n_blocks128 + nb] = sc;
          }
          fence_proxy_async_smem();
          named_bar_sync(1, kPairEpiThreads);
          if (et == 0) {
            if (ok && !ctx.aborted && row0 < p.m) {
              tma_store_2d(&outs[0], hand + 2 * kTileOutHalfBytes, nb * kTileN, row0);
              tma_store_commit();
              tma_store_wait_read0();
            }
            mbar_arrive(bar_hand_empty);
          }
        } else {
        if (last_tile) {
          pair_swiglu_chunks(hand_gen, et, kPairAllHands);  // shared with the consumer warps
          fence_proxy_async_smem();
          named_bar_sync(4, kPairAllHands);
        } else {
#if !(defined(GU_EXP) && GU_EXP == 9)  // (experiment 9: the epilogue warps store the gate tile without the SwiGLU arithmetic)
          pair_swiglu_chunks(hand_gen, et, kPairEpiThreads);
#endif
          fence_proxy_async_smem();
          named_bar_sync(1, kPairEpiThreads);
        }
        if (et == 0) {
          if (ok && !ctx.aborted && row0 < p.m &&
              GU_IN_RANGE(p.out_cols == 0 || (nb * kTileN + 128 <= p.out_cols && row0 >= 0 && row0 < p.out_rows),
                          kSitePairStore)) {
            if constexpr (kMode == kPairGather) {
              // Destinations are visited in a rotation that differs per source rank and per cluster, so that at any
              // moment the box's ranks are writing to different peers instead of all to the same one.
              const int peers = p.out_count - 1;
              const int col = p.out_col0 + nb * kTileN;
              tma_store_2d(&outs[p.out_rank], hand, col, row0);
              tma_store_2d(&outs[p.out_rank], hand + kTileOutHalfBytes, col + 64, row0);
              for (int i = 0; i < peers; ++i) {
                const int hop = 1 + (i + cluster_id + pm) % peers;
                const CUtensorMap* dst = &outs[(p.out_rank + hop) % p.out_count];
                tma_store_2d(dst, hand, col, row0);
                tma_store_2d(dst, hand + kTileOutHalfBytes, col + 64, row0);
              }
            } else {
              tma_store_2d(&outs[0], hand, nb * kTileN, row0);
              tma_store_2d(&outs[0], hand + kTileOutHalfBytes, nb * kTileN + 64, row0);
            }
            tma_store_commit();
            tma_store_wait_read0();  // the tile may be overwritten once the stores have read it
          }
          mbar_arrive(bar_hand_empty);
        }
        }
        GU_TR_END(7);
        hand_phase ^= 1u;
      }
      if (et == 0) tma_store_wait_all0();
    }
  } else {
    reg_alloc<kPairConsumerRegs>();
    // ------------------------------- consumers --------------------------------
    // Warps 4-7 promote the gate half of every K block, warps 8-11 the up half: a thread owns one token row and all
    // 128 columns of one projection.
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const uint32_t proj = static_cast<uint32_t>(warp - 4) >> 2;  // 0: gate, 1: up
    const int row = quarter * 32 + lane;   // token row inside this CTA's 128
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + proj * kTileN;
    const uint32_t stage_free_even = mapa_shared(bar_stage_free, 0);
    const float* scale_w = (proj && !kSingle) ? p.scale_up : p.scale_gate;
    uint32_t blocks_done = 0;  // K blocks walked so far: accumulator stage = bit 0, ring stage = low bits, phases above
    uint32_t hand_phase = 0;

    PairWalk<kStreamK> walk(p, cluster_id, clusters);
    int tile = 0, jb = 0, je = 0;
    bool have = walk.next(p, tile, jb, je);
    // stream-K: this launch's stamp (never 0) and this CTA's hand-off slot: [256 columns][128 rows] fp32
    unsigned int epoch = 0;
    // (stream-K) consumer thread 0 fetches the stamp the first epilogue thread left in shared memory
    auto fetch_epoch = [&]() {
      const unsigned long long t0 = globaltimer_ns();
      while ((epoch = *epoch_gen) == 0u) {
        spin_backoff_ns(64u);
        if (globaltimer_ns() - t0 > g_wait_limit_ns) {
          ctx.fail(kWaitPairFlag, (kWaitPairFlag << 24) | (blockIdx.x & 0xffffffu));
          break;
        }
      }
    };
    // element offsets of this thread's scale rows (the host keeps M * K/128 and N/128 * K/128 below 2^31)
    uint32_t sx_off = 0, sw_off = 0;
    float sx0 = 0.f, sw0 = 0.f;
    // first scales of a segment (fetched before the previous tile is handed over)
    auto start_tile = [&](int t, int j0) {
      int pm, nb;
      tile_coords(p, t, pm, nb);
      const int m_global = min((2 * pm + static_cast<int>(rank)) * kTileM + row, p.m - 1);
      sx_off = static_cast<uint32_t>(m_global) * static_cast<uint32_t>(p.kb);
      const int wblock = kSingle ? min(2 * nb + static_cast<int>(proj), p.n_blocks128 - 1) : nb;
      sw_off = static_cast<uint32_t>(wblock) * static_cast<uint32_t>(p.kb);
      if (!GU_IN_RANGE(m_global >= 0 && m_global < p.m && wblock >= 0 &&
                           wblock < (kSingle ? p.n_blocks128 : p.num_n_blocks), kSitePairScale))
        return;
      sx0 = __ldg(p.scale_x + sx_off + j0);
      sw0 = __ldg(scale_w + sw_off + j0);
    };
    if (have) start_tile(tile, jb);
#ifdef GU_TRACE
    bool tr_first = true, tr_seen = false;
#endif

    while (have) {
#ifdef GU_TRACE
      tr_first = !tr_seen;
      tr_seen = true;
#endif
      float2 sums[64];       // this row's 128 running sums of one projection
      // piece buffers: one round (kPairInFlight pieces) is being added while the next round's loads are in flight
      float va[kPairPiece], vb[kPairPiece], vc[kPairInFlight == 2 ? kPairPiece : 1], vd[kPairInFlight == 2 ? kPairPiece : 1];
#pragma unroll
      for (int i = 0; i < 64; ++i) sums[i] = make_float2(0.f, 0.f);
#if defined(GU_EXP) && GU_EXP == 6
#pragma unroll
      for (int i = 0; i < kPairPiece; ++i) {
        va[i] = vb[i] = 1.f;
        if (kPairInFlight == 2) vc[i] = vd[i] = 1.f;
      }
#endif
#ifdef GU_TRACE
      const unsigned long long tr_loop0 = clock64();
#endif
      for (int j = jb; j < je; ++j) {
        // the next K block's scales are fetched one block ahead of their use
        float sx1 = 0.f, sw1 = 0.f;
        if (j + 1 < je) {
          sx1 = __ldg(p.scale_x + sx_off + j + 1);
          sw1 = __ldg(scale_w + sw_off + j + 1);
        }
        const float sc = sx0 * sw0;
        const float2 scv = make_float2(sc, sc);
        const uint32_t acc = blocks_done & 1u;
        const uint32_t stage = blocks_done % kPairStages, phase = (blocks_done / kPairStages) & 1u;
        const uint32_t t = lane_addr + acc * (2 * kTileN);

        // This half's 128 columns come in pieces of kPairPiece columns through four buffers; the stage goes back to the
        // issuer as soon as the last piece is in registers.  (Loads of 16 columns instead of 32: same registers, but
        // the allocator places four 16-register blocks without spilling, two 32-register ones not.)
        GU_TR_BEGIN();
        mbar_wait_lane(ctx, lane == 0, bar_done + 8 * stage, phase, kWaitPairDone);
        GU_TR_END(3);
        GU_EV(1, j, 0);
        tc_fence_after();
        pair_ld(t, va);
        if constexpr (kPairInFlight == 2) pair_ld(t + kPairPiece, vb);
#if defined(GU_EXP) && (GU_EXP == 7 || GU_EXP == 8)
        // experiments: only 64 of the 128 columns are read (two rounds of loads instead of four) before the stage goes
        // back; 7 still does the arithmetic of all 128 columns (on stale registers), 8 only that of the 64
        tmem_ld_wait_pin<kPairPiece>(va);
        tmem_ld_wait_pin<kPairPiece>(vb);
        pair_ld(t + 2 * kPairPiece, vc);
        pair_ld(t + 3 * kPairPiece, vd);
        pair_fma(sums, va, scv);
        pair_fma(sums + 8, vb, scv);
        tmem_ld_wait_pin<kPairPiece>(vc);
        tmem_ld_wait_pin<kPairPiece>(vd);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(stage_free_even + 8 * acc);
        pair_fma(sums + 16, vc, scv);
        pair_fma(sums + 24, vd, scv);
#if GU_EXP == 7
        pair_fma(sums + 32, va, scv);
        pair_fma(sums + 40, vb, scv);
        pair_fma(sums + 48, vc, scv);
        pair_fma(sums + 56, vd, scv);
#endif
#elif defined(GU_EXP) && GU_EXP == 10
        // experiment: 64 of the 128 columns are read in one batch, the stage goes back at once, all the arithmetic of
        // 128 columns follows (on stale registers for the second half): what consumers with half the columns each
        // and twice the warps could reach at most
        pair_ld(t + 2 * kPairPiece, vc);
        pair_ld(t + 3 * kPairPiece, vd);
        tmem_ld_wait();
        pin_regs<kPairPiece>(va);
        pin_regs<kPairPiece>(vb);
        pin_regs<kPairPiece>(vc);
        pin_regs<kPairPiece>(vd);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(stage_free_even + 8 * acc);
        pair_fma(sums, va, scv);
        pair_fma(sums + 8, vb, scv);
        pair_fma(sums + 16, vc, scv);
        pair_fma(sums + 24, vd, scv);
        pair_fma(sums + 32, va, scv);
        pair_fma(sums + 40, vb, scv);
        pair_fma(sums + 48, vc, scv);
        pair_fma(sums + 56, vd, scv);
#elif GU_PIECE == 16 && GU_INFLIGHT == 2 && !defined(GU_CONSUMER_ROUNDS)
        // The shipped schedule: all four buffers are filled at once (64 columns in flight), each pair is refilled as
        // soon as it has been added, and the stage goes back when the second 64 columns are in registers — two load
        // latencies and 32 packed FMAs on the way to the release.  (The round-by-round loop below, four latencies:
        // 0.433 against 0.4255 ms on prefill_8b.)
        pair_ld(t + 2 * kPairPiece, vc);
        pair_ld(t + 3 * kPairPiece, vd);
        tmem_ld_wait();
        pin_regs<kPairPiece>(va);
        pin_regs<kPairPiece>(vb);
        pin_regs<kPairPiece>(vc);
        pin_regs<kPairPiece>(vd);
        pair_fma(sums, va, scv);
        pair_fma(sums + 8, vb, scv);
        pair_ld(t + 4 * kPairPiece, va);
        pair_ld(t + 5 * kPairPiece, vb);
        pair_fma(sums + 16, vc, scv);
        pair_fma(sums + 24, vd, scv);
        pair_ld(t + 6 * kPairPiece, vc);
        pair_ld(t + 7 * kPairPiece, vd);
        tmem_ld_wait();
        pin_regs<kPairPiece>(va);
        pin_regs<kPairPiece>(vb);
        pin_regs<kPairPiece>(vc);
        pin_regs<kPairPiece>(vd);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(stage_free_even + 8 * acc);  // the half is in registers: hand it back
        GU_EV(1, j, 3);
        pair_fma(sums + 32, va, scv);
        pair_fma(sums + 40, vb, scv);
        pair_fma(sums + 48, vc, scv);
        pair_fma(sums + 56, vd, scv);
#else
        // Round by round (the other piece sizes, one load in flight, and -DGU_CONSUMER_ROUNDS): kPairInFlight pieces
        // per round through two alternating sets of buffers, the loads of a round in flight while the round before
        // it is added.
#pragma unroll
        for (int q = 0; q < kPairRounds; ++q) {
          // buffers of this round and of the next (one or two pieces each)
          float* c0 = (kPairInFlight == 2) ? ((q & 1) ? vc : va) : ((q & 1) ? vb : va);
          float* c1 = (q & 1) ? vd : vb;
          float* n0 = (kPairInFlight == 2) ? ((q & 1) ? va : vc) : ((q & 1) ? va : vb);
          float* n1 = (q & 1) ? vb : vd;
          tmem_ld_wait_pin<kPairPiece>(c0);
          if constexpr (kPairInFlight == 2) tmem_ld_wait_pin<kPairPiece>(c1);
          if (q + 1 < kPairRounds) {
            pair_ld(t + (q + 1) * kPairInFlight * kPairPiece, n0);
            if constexpr (kPairInFlight == 2) pair_ld(t + ((q + 1) * 2 + 1) * kPairPiece, n1);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(stage_free_even + 8 * acc);  // the half is in registers: hand it back
            GU_EV(1, j, 3);
          }
          // The round before the last is not added until the last round is in registers too, so that the stage goes
          // back one round of arithmetic earlier (both rounds sit in the two buffer sets meanwhile).
          if (q + 2 != kPairRounds) {
            pair_fma(sums + q * kPairInFlight * (kPairPiece / 2), c0, scv);
            if constexpr (kPairInFlight == 2) pair_fma(sums + (q * 2 + 1) * (kPairPiece / 2), c1, scv);
          }
          if (q + 1 == kPairRounds) {
            pair_fma(sums + (q - 1) * kPairInFlight * (kPairPiece / 2), n0, scv);
            if constexpr (kPairInFlight == 2) pair_fma(sums + ((q - 1) * 2 + 1) * (kPairPiece / 2), n1, scv);
          }
        }
#endif

        ++blocks_done;
        sx0 = sx1;
        sw0 = sw1;
      }
#ifdef GU_TRACE
      if (tr_me) {
        atomicAdd(&g_trace[blockIdx.x & 1][5], (unsigned long long)(clock64() - tr_loop0));
        atomicAdd(&g_trace[blockIdx.x & 1][10], (unsigned long long)(je - jb));
      }
#endif

      // next segment's coordinates and first scales, so their latency hides under the hand-over
      int next_tile = 0, next_jb = 0, next_je = 0;
      const bool have_next = walk.next(p, next_tile, next_jb, next_je);
      if (have_next) start_tile(next_tile, next_jb);

      if constexpr (kStreamK) {
        const int ct = static_cast<int>(threadIdx.x) - 128;  // 0 .. 255 over the consumer warps
        if (jb != 0) {
          // -------- the remainder of a tile the cluster before this one owns: publish the running sums --------
          // slot of this CTA: [32][256 consumer threads] float4, values 4i .. 4i+3 of thread t at [i * 256 + t]
          float4* slot = reinterpret_cast<float4*>(p.partials + static_cast<size_t>(blockIdx.x) * kTilePartialFloats) + ct;
          if (GU_IN_RANGE(blockIdx.x < static_cast<unsigned>(kPairMaxCtas), kSitePairHandOff)) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              __stcg(slot + i * 256, make_float4(sums[2 * i].x, sums[2 * i].y, sums[2 * i + 1].x, sums[2 * i + 1].y));
          }
          __threadfence();
          named_bar_sync(3, 256);
          if (ct == 0) {
            if (epoch == 0u) fetch_epoch();
            if (!ctx.aborted) st_release_gpu(p.flags + kPairFlagWord0 + blockIdx.x, epoch);
          }
          tile = next_tile; jb = next_jb; je = next_je; have = have_next;
          continue;
        }
        if (je != p.kb) {
          // -------- owner of a tile whose last K blocks the next cluster walked: add its sums --------
          const unsigned int peer_cta = blockIdx.x + 2u;  // same rank, next cluster
          if (ct == 0 && epoch == 0u) fetch_epoch();
          if (ct == 0 && !ctx.aborted) {
            unsigned long long t0 = 0;
            for (uint32_t it = 1; ld_acquire_gpu(p.flags + kPairFlagWord0 + peer_cta) != epoch; ++it) {
              spin_backoff_ns(64u);
              if ((it & 255u) == 0u) {
                const unsigned long long now = globaltimer_ns();
                if (t0 == 0) {
                  t0 = now;
                } else if (now - t0 > g_wait_limit_ns || ctx.raised()) {
                  ctx.fail(kWaitPairFlag, (kWaitPairFlag << 24) | (blockIdx.x & 0xffffffu));
                  break;
                }
              }
            }
          }
          named_bar_sync(3, 256);
          if (!ctx.raised() && GU_IN_RANGE(peer_cta < gridDim.x, kSitePairHandOff)) {
            const float4* slot =
                reinterpret_cast<const float4*>(p.partials + static_cast<size_t>(peer_cta) * kTilePartialFloats) + ct;
#pragma unroll
            for (int half = 0; half < 2; ++half) {  // 16 loads of 16 bytes in flight (the piece buffers are free here)
              float4 buf[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) buf[i] = __ldcg(slot + (16 * half + i) * 256);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float4 v = buf[i];
                sums[2 * (16 * half + i)].x += v.x;
                sums[2 * (16 * half + i)].y += v.y;
                sums[2 * (16 * half + i) + 1].x += v.z;
                sums[2 * (16 * half + i) + 1].y += v.w;
              }
            }
          }
        }
      }

      // -------- hand-over: this projection's bf16 tile in the output staging layout (two 64-column half tiles of
      // 128-byte rows, 16-byte chunks swizzled by the row) --------
      GU_TR_BEGIN();
      mbar_wait_lane(ctx, lane == 0, bar_hand_empty, hand_phase ^ 1u, kWaitPairHandEmpty);
      {
        uint8_t* tile_row = smem_gen + (hand - smem_base) + proj * (2 * kTileOutHalfBytes) + row * 128;
#pragma unroll
        for (int c = 0; c < 16; ++c) {  // 16 chunks of 8 bf16 = 16 bytes
          uint4 q;
          q.x = pack_bf16x2(sums[4 * c + 0].x, sums[4 * c + 0].y);
          q.y = pack_bf16x2(sums[4 * c + 1].x, sums[4 * c + 1].y);
          q.z = pack_bf16x2(sums[4 * c + 2].x, sums[4 * c + 2].y);
          q.w = pack_bf16x2(sums[4 * c + 3].x, sums[4 * c + 3].y);
          *reinterpret_cast<uint4*>(tile_row + (c >> 3) * kTileOutHalfBytes + (((c & 7) ^ (row & 7)) << 4)) = q;
        }
      }
      if constexpr (kSingle) fence_proxy_async_smem();  // these bytes are read by the TMA stores as they are
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_hand_full);
      GU_TR_END(6);
      if constexpr (kShareLast) {
        if (!have_next) {
          // this cluster's last tile: once all eight warps' halves are in, share its SwiGLU with the epilogue warps
          GU_TR_BEGIN();
          mbar_wait_lane(ctx, lane == 0, bar_hand_full, hand_phase, kWaitPairHandFull);
          GU_TR_END(11);
          GU_TR_BEGIN();
          pair_swiglu_chunks(smem_gen + (hand - smem_base), kPairEpiThreads + static_cast<int>(threadIdx.x) - 128,
                             kPairAllHands);
          fence_proxy_async_smem();
          GU_TR_END(12);
          GU_TR_BEGIN();
          named_bar_sync(4, kPairAllHands);
          GU_TR_END(13);
        }
      }
      hand_phase ^= 1u;
      tile = next_tile; jb = next_jb; je = next_je; have = have_next;
    }
  }

  // ------------------------------- teardown --------------------------------
  if (*abort_gen) {
    // give copies that were already in flight time to land before shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) spin_backoff_ns(1000u);
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();  // neither CTA leaves while the other may still reach into it
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, kTileTmemCols);
  }
#ifdef GU_TRACE
  if (blockIdx.x < 2 && threadIdx.x == 0) atomicAdd(&g_trace[blockIdx.x & 1][9], (unsigned long long)(clock64() - tr_cta0));
#endif
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gateup_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                   const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_out,
                   const TileParams p) {
  pair_kernel_body<false>(tm_x, tm_gate, tm_up, &tm_out, p);
}

// The same with the stream-K schedule (see PairWalk; needs TileParams::flags / partials).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gateup_pair_sk_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                      const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_out,
                      const TileParams p) {
  pair_kernel_body<false, kPairPlain, true>(tm_x, tm_gate, tm_up, &tm_out, p);
}

// Gate/up + SwiGLU with the column all-gather fused into the epilogue (see TileParams::out_count).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gateup_pair_gather_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                          const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ PeerMaps peers,
                          const TileParams p) {
  pair_kernel_body<false, kPairGather>(tm_x, tm_gate, tm_up, peers.m, p);
}

// Gate/up + SwiGLU with the result re-quantised to e4m3 + 1x128 scales in the epilogue; `tm_outq` describes the
// e4m3 [M, N] destination with 128-byte x 128-row boxes.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gateup_pair_fp8out_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gate,
                          const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ CUtensorMap tm_outq,
                          const TileParams p) {
  pair_kernel_body<false, kPairFp8Out>(tm_x, tm_gate, tm_up, &tm_outq, p);
}

// Plain block-scaled GEMM (single-projection mode) on CTA pairs.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
blockwise_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_c, const TileParams p) {
  pair_kernel_body<true>(tm_a, tm_b, tm_b, &tm_c, p);
}

// Plain block-scaled GEMM whose output tiles are scattered to the ranks that own their token rows (see
// TileParams::blocks_per_owner): the compute half of a fused GEMM + reduce-scatter.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
blockwise_gemm_pair_scatter_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                                   const __grid_constant__ PeerMaps peers, const TileParams p) {
  pair_kernel_body<true, kPairScatter>(tm_a, tm_b, tm_b, peers.m, p);
}

}  // namespace gu
