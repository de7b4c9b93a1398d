/*
 * C ABI of the B200 FP8 gate/up-projection + SwiGLU library (libgateup.so).
 *
 *   output[M, N] (bf16) = SiLU(X . Wg^T) * (X . Wu^T)
 *
 * X is e4m3 [M, K] with fp32 scales [M, K/128]; Wg / Wu are e4m3 [N, K] with
 * fp32 scales [N/128, K/128]; all row-major and contiguous (output may have a
 * row pitch larger than N).  These are the tensors the reference entry point
 * takes, in its order:
 *   kernels/179_fp8_mlp_gate_up_projection/kernel.py:398-407            (Python `run`)
 *   kernels/179_fp8_mlp_gate_up_projection/variants/cuda_cpp_v4/binding.cpp:18-25 (pybind `run`)
 *
 * Every pointer is a device pointer on the current device, 16-byte aligned.
 * No entry point allocates or frees device memory; scratch is passed in by the
 * caller (gu_run_decode_static carries its own).  All launches go to the stream that is passed in.  Functions return 0
 * on success or a negative GU_E* code; nothing throws.
 */
#ifndef GATEUP_H_
#define GATEUP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GU_VERSION 1

/* error codes */
#define GU_OK 0
#define GU_EINVAL_NULL (-1)      /* a required pointer is null                         */
#define GU_EINVAL_SHAPE (-2)     /* M < 1, or K or N not a positive multiple of 128    */
#define GU_EINVAL_ALIGN (-3)     /* a pointer or the output pitch is not 16-B aligned  */
#define GU_EINVAL_PLAN (-4)      /* unknown plan id, or the plan cannot run this shape */
#define GU_EWORKSPACE (-5)       /* workspace missing or smaller than required         */
#define GU_ECUDA (-6)            /* a CUDA runtime / driver call failed                */
#define GU_EDEVICE (-7)          /* not a compute-capability-10.x device               */
#define GU_ETIMEOUT (-8)         /* a bounded device-side wait gave up (gu_last_status) */
#define GU_ESTATIC_LIMIT (-9)    /* gu_run_decode_static: more tokens than its built-in scratch holds */
#define GU_EBOUNDS (-10)         /* range-checked debug build only: an index or coordinate left its extent (gu_last_status) */

/* plans */
#define GU_PLAN_AUTO 0    /* shape heuristic (gu_select_plan)                                      */
#define GU_PLAN_TILE 1    /* persistent tiles of both projections; any M; above 128 tokens CTA pairs or lone CTAs,
                             whichever the tile counts favour (same bits for whole tiles) */
#define GU_PLAN_STREAM 2  /* weight-streaming, tokens on the MMA N side, stream-K over (N-block, K-block); M <= 64 */
#define GU_PLAN_TILE_DP 3 /* lone-CTA tile kernel, data-parallel schedule forced (whole tiles per CTA, no scratch) */
#define GU_PLAN_TILE_SK 4 /* lone-CTA tile kernel, stream-K schedule forced (needs scratch)                  */
#define GU_PLAN_TILE_PAIR 5      /* CTA-pair tile kernel forced (256-token tiles, cta_group::2), any M, whole tiles per cluster */
#define GU_PLAN_TILE_PAIR_SK 6   /* CTA-pair tile kernel, stream-K schedule forced (needs scratch; at least as many
                                    256-token x 128-column tiles as CTA pairs on the device, else GU_EINVAL_PLAN) */

/*
 * One call's operands.  Replaces the seven tensors of the reference `run`
 * (kernel.py:398-407) plus what its host glue derives from them: M, K, N
 * (kernel.py:354,419) and the launch stream (kernel.py:212-213, passed to
 * gu_run separately).
 */
typedef struct gu_problem {
  const void* x;            /* e4m3 [M, K]                 */
  const float* scale_x;     /* f32  [M, K/128]             */
  const void* gate_w;       /* e4m3 [N, K]                 */
  const float* scale_gate;  /* f32  [N/128, K/128]         */
  const void* up_w;         /* e4m3 [N, K]                 */
  const float* scale_up;    /* f32  [N/128, K/128]         */
  void* output;             /* bf16 [M, ld_output], columns [0, N) written */
  int64_t m, k, n;
  int64_t ld_output;        /* row pitch of output in elements (>= N, multiple of 8) */
  void* workspace;          /* gu_workspace_bytes() bytes, prepared once by gu_workspace_init; may be null when 0 */
  size_t workspace_bytes;
  int32_t plan;             /* GU_PLAN_*                   */
  int32_t reserved;
} gu_problem;

/* Library version (GU_VERSION). */
int gu_version(void);

/* Static message for a GU_E* code. */
const char* gu_error_string(int code);

/*
 * Tile / split policy.  Stands where the reference has `_select_config`
 * (kernel.py:232-249) and the even/odd-M dispatch of `launch_fp8_mlp_gate_up`
 * (variants/cuda_cpp_v4/kernel.cu:297-311).  Returns GU_PLAN_TILE or
 * GU_PLAN_STREAM for a valid shape, or a negative code.
 */
int gu_select_plan(int64_t m, int64_t k, int64_t n);

/*
 * Which tile kernel and schedule the tile plan runs for `op` on this shape on
 * the current device (148 SMs assumed when there is none): GU_PLAN_TILE_DP
 * (lone CTAs, whole tiles), GU_PLAN_TILE_SK, GU_PLAN_TILE_PAIR or
 * GU_PLAN_TILE_PAIR_SK; `with_workspace` says whether the call will pass
 * scratch (the stream-K schedules need it; only GU_OP_GATEUP has them).  The
 * reference's counterpart is the parity test on M / 128 in
 * `launch_fp8_mlp_gate_up` (variants/cuda_cpp_v4/kernel.cu:297-311), which
 * picks its 2-CTA or 1-CTA configuration; here the choice follows measured
 * costs (rounds of tiles x max(K blocks per tile, epilogue length)).  Whole
 * tiles give the same bits on either kernel.  Returns a negative code for a
 * shape or `op` that is not supported.
 */
#define GU_OP_GATEUP 0     /* gu_run / gu_run_concat */
#define GU_OP_GATEUP_FP8 1 /* gu_run_fp8out */
#define GU_OP_GEMM 2       /* gu_blockwise_gemm */
int gu_select_tile_kernel(int op, int64_t m, int64_t k, int64_t n, int with_workspace);

/*
 * Scratch bytes a plan needs for this shape (0 when it needs none).  The
 * reference allocates its scratch inside the call (kernel.py:226-229,
 * cuda_cpp_v4/kernel.cu:221-230, 290-296); here the caller owns it.
 */
size_t gu_workspace_bytes(int64_t m, int64_t k, int64_t n, int plan);

/*
 * Prepare freshly allocated scratch (zeroes the hand-off flags; enqueued on
 * `stream`).  Needed once per allocation, not per call: each launch stamps the
 * flags with a new epoch, taken from a launch counter inside the workspace.
 * Calls that share one workspace must not overlap on the GPU.
 */
int gu_workspace_init(void* workspace, size_t bytes, void* stream);

/*
 * Launch the fused op on `stream` (a cudaStream_t).  Replaces the whole body
 * of the reference `run`: two GEMM launches and the SwiGLU launch
 * (kernel.py:487-503), or `launch_fp8_mlp_gate_up` (cuda_cpp_v4/kernel.cu:271-341).
 * Asynchronous; returns after the launch with 0 or a negative code.
 * With GU_PLAN_AUTO / TILE / TILE_DP / TILE_PAIR / TILE_PAIR_SK / STREAM the
 * launch keeps no host-side state (the stream-K schedules of the pair and the
 * streaming kernel count their launches in the workspace), so a launch recorded
 * in a CUDA graph may be replayed (the workspace must stay allocated and be used
 * by nothing else meanwhile); GU_PLAN_TILE_SK, a study option, stamps its flags
 * from a host counter and must not be replayed.
 * GU_PLAN_TILE above 128 tokens picks the pair kernel's stream-K schedule when a
 * workspace of gu_workspace_bytes() is passed, there are at least two rounds of
 * tiles and whole tiles would leave 10 % or more of the device idle in the last; the sums of a tile cut in two are
 * joined by one extra fp32 addition, so its outputs may differ from the
 * data-parallel schedule's in the last bf16 digit.  Without a workspace the
 * data-parallel schedule runs.
 */
int gu_run(const gu_problem* problem, void* stream);

/*
 * Same op with concatenated weights W[2N, K] (gate rows first) and scales
 * [2N/128, K/128]; slices and forwards to gu_run.
 */
int gu_run_concat(const void* x, const float* scale_x, const void* w2n, const float* scale_w2n,
                  void* output, int64_t m, int64_t k, int64_t n, int64_t ld_output,
                  void* workspace, size_t workspace_bytes, int plan, void* stream);

/*
 * Column-parallel variant with the all-gather fused into the epilogue.  `problem` describes this
 * rank's shard (n = N / world columns; `output`, `workspace`, `plan` are ignored); `rank_outputs[r]`
 * is rank r's full bf16 [M, ld_full] buffer (N = n * world columns) mapped into this process (its own
 * buffer for r == rank, peers' buffers through CUDA peer / symmetric-memory mappings).  Every output
 * tile is written by plain TMA stores into all `world` buffers at column offset rank * n, so after
 * all ranks' launches have completed (a cross-rank barrier is the caller's job) every rank holds the
 * contiguous [M, N] result.  world <= 8.  No load ever touches peer memory.  The reference is
 * single-GPU and has no counterpart; it stands where an NCCL all-gather + permute would follow gu_run.
 */
int gu_run_gather(const gu_problem* problem, void* const* rank_outputs, int world, int rank, int64_t ld_full,
                  void* stream);

/*
 * gu_run with the result re-quantised in the epilogue: out_q[M, N] e4m3 (contiguous) and out_scale[M, N/128]
 * fp32, scale = amax over the token's 128 columns / 448 — the operand format of the next block-scaled GEMM
 * (gu_blockwise_gemm as the down projection), so the bf16 intermediate never reaches HBM.  Bits equal
 * quantising gu_run's bf16 result with gu_quantize_activation.  `output`, `workspace` and `plan` of the
 * problem are ignored.  No counterpart in the reference, whose path ends at the bf16 result.
 */
int gu_run_fp8out(const gu_problem* problem, void* out_q, float* out_scale, void* stream);

/*
 * Plain block-scaled FP8 GEMM:  c[M, N] (bf16, row pitch ld_c) = sum over K blocks of
 * scale_a[m, kb] * scale_b[n/128, kb] * (a[m, kb] . b[n, kb]^T), a e4m3 [M, K] with fp32 scales [M, K/128],
 * b e4m3 [N, K] with fp32 scales [N/128, K/128].  This is the GEMM the reference launches twice per call
 * (NVIDIA's BlockwiseGemmKernel, loaded at kernel.py:43-72 and launched at kernel.py:487-488; CUTLASS
 * builder form at variants/cuda_cpp_v4/kernel.cu:185-233), run by the same tile kernel in
 * single-projection mode.  It serves the MLP's down projection.  One launch on `stream`.
 */
int gu_blockwise_gemm(const void* a, const float* scale_a, const void* b, const float* scale_b, void* c, int64_t m,
                      int64_t k, int64_t n, int64_t ld_c, void* stream);

/*
 * Row-parallel block-scaled GEMM with the reduce-scatter fused into its epilogue — first half of a fused
 * GEMM + all-reduce over `world` GPUs of one box (the MLP's down projection when the intermediate dimension
 * is sharded).  This rank multiplies a[M, K_local] by b[N, K_local]^T (same operand formats as
 * gu_blockwise_gemm) and stores every bf16 partial tile with a plain TMA store straight into the buffer of
 * the rank that owns those token rows: rank r owns rows [r*M/world, (r+1)*M/world); rank_slots[r] is r's
 * buffer [world][M/world][N] bf16 as mapped into this process (symmetric memory / CUDA peer mapping), and
 * this rank writes slot `rank` of it.  M must be a multiple of 128 * world.  No load touches peer memory.
 * The caller runs a cross-rank barrier, then gu_reduce_gather.  The reference is single-GPU: no counterpart.
 */
int gu_blockwise_gemm_scatter(const void* a, const float* scale_a, const void* b, const float* scale_b,
                              void* const* rank_slots, int world, int rank, int64_t m, int64_t k, int64_t n,
                              void* stream);

/*
 * Second half: sums this rank's `world` slots ([world][M/world][H] bf16, filled by all ranks'
 * gu_blockwise_gemm_scatter) in rank order in fp32, rounds once to bf16 and writes the reduced rows into
 * every rank's full result rank_outputs[r] ([M][H] bf16, contiguous) at row rank*M/world, with 16-byte
 * stores (over NVLink for the peers); a null rank_outputs[r] other than this rank's own is skipped, which with
 * all peers null is the reduce-scatter form (each rank keeps only its own rows).  After a second cross-rank
 * barrier every rank holds the full sum.
 * The summation order is fixed, so all ranks hold identical bits.  H a multiple of 8.  No counterpart in the
 * reference; it stands where an NCCL all-reduce would follow gu_blockwise_gemm.
 */
int gu_reduce_gather(const void* slots, void* const* rank_outputs, int world, int rank, int64_t m, int64_t h,
                     void* stream);

/*
 * Cross-rank barrier for the fused gather / reduce entry points above, enqueued on `stream`: a one-warp kernel in
 * which this rank stamps its slot in every rank's flag array (plain stores, over NVLink for the peers) and then
 * polls its OWN array until all `world` slots carry the stamp; everything this rank's earlier launches on the
 * stream wrote to peer memory is visible to a peer once that peer has passed the barrier.  rank_flags[r] is rank r's
 * flag array as mapped into this process: 64 uint32 of symmetric / peer-mapped memory, zeroed once (with a host-side
 * barrier after the zeroing) before the first use and touched by nothing else.  Every rank must call it the same
 * number of times.  The wait is bounded: after `limit_ns` nanoseconds (0: 2 s) the kernel gives up, gu_last_status
 * reports GU_ETIMEOUT with wait id 20 and the index of a rank that did not arrive, and the context stays usable —
 * where the reference's only cross-CTA wait spins without bound (blockwise_gemm_fused.py:85-91).  No load touches
 * peer memory, nothing is multicast.  The reference is single-GPU: no counterpart.
 */
int gu_peer_barrier(void* const* rank_flags, int world, int rank, uint64_t limit_ns, void* stream);

/*
 * Activation quantiser, the step in front of gu_run: x[M, K] (bf16, or fp32 when x_is_f32 != 0; row pitch ld_x
 * elements) -> q[M, K] e4m3 and scale[M, K/128] fp32 with scale = amax of the 1x128 block / 448, the layout
 * `x` / `scale_x` of gu_problem.  The reference takes its activations already quantised
 * (kernel.py:356-357), so it has no counterpart; the bits equal PyTorch's
 * clamp(x / scale, -448, 448).to(float8_e4m3fn).  One streaming launch on `stream`.
 */
int gu_quantize_activation(const void* x, int x_is_f32, int64_t ld_x, void* q, float* scale, int64_t m, int64_t k,
                           void* stream);

/*
 * Device-side status of the current device: 0, or GU_ETIMEOUT with `detail`
 * = (wait id << 24 | block index) of the first wait that gave up (or, from the
 * range-checked debug build, GU_EBOUNDS with detail = site << 16 | block).  Synchronises
 * the device; meant for tests and debugging, never for the timed path.  The
 * reference has no counterpart (its cluster wait spins without bound,
 * variants/cute_fused_v1/blockwise_gemm_fused.py:85-91).  `clear` != 0 resets it.
 */
int gu_last_status(int* detail, int clear);

/*
 * 1 if this library was built with -DGU_BOUNDS=1, the range-checked debug build that stands in for a memory
 * checker: every computed TMA coordinate, global index and ring / accumulator stage index of the kernels is tested
 * against its extent before use, a violation is recorded (gu_last_status returns GU_EBOUNDS with detail =
 * site << 16 | block) and the access is skipped.  0 for the regular library, where the tests compile to nothing.
 * No counterpart in the reference.
 */
int gu_is_range_checked_build(void);

/*
 * Decode-sized variant of gu_run for callers that cannot hand the library any
 * scratch memory because they are not allowed to allocate on the device: a
 * plugin inside a serving runtime that claims all of HBM for its own arena at
 * start-up and forbids cudaMalloc afterwards, or a latency-critical decode loop
 * that cannot afford the device-wide synchronisation a cudaMalloc / cudaFree
 * implies.  It runs the weight-streaming (stream-K) kernel with its hand-off
 * scratch in an array compiled into the library (4 MiB + 4 KiB on every GPU
 * that loads the library, held until the process exits) and calls no
 * cudaMalloc, cudaFree or other allocating routine.  The caller still passes
 * inputs and output; `workspace`, `workspace_bytes` and `plan` are ignored.
 *
 *   - At most 16 tokens (M <= 16).  A larger M returns GU_ESTATIC_LIMIT and
 *     launches nothing.
 *   - The first call on each device looks up the array's device address and
 *     sets the kernel's shared-memory attribute.  Make that call with the
 *     device current, and before any stream capture begins.  That first call
 *     (or, with lazy module loading, the first launch of any kernel of this
 *     library) is also what loads the module onto the device: its code plus
 *     the 4 MiB + 4 KiB array.  A host that claims all of HBM for an arena
 *     of its own must therefore make this call — or load the library with
 *     CUDA_MODULE_LOADING=EAGER and touch the device — BEFORE it claims the
 *     arena; GU_ECUDA from the first call most likely means that the module
 *     load found no memory left.
 *   - Every call this process makes on a device uses the same array, and the
 *     array keeps what the previous call left in it.  Nothing has to be
 *     cleared between calls (each call stamps its hand-off flags with an epoch
 *     no earlier call used), but two calls in flight on the GPU at the same
 *     time — two streams, or two host threads — race on it and give wrong
 *     results.  Keep these calls on one stream.
 *
 * This entry point has no counterpart in the reference, which allocates its
 * scratch inside every call.
 */
int gu_run_decode_static(const gu_problem* problem, void* stream);

/*
 * Numerical notes that hold for every entry point above.  The activation is computed as g / (1 + exp(-g)) with
 * the hardware's approximate division: for gate values between about -88.7 and -87.3 (denominator in
 * (2^126, 2^128)) that division returns 0 where g * sigmoid(g) would be a normal number of magnitude ~1e-36 — a
 * deviation of that size and nothing more.  gu_quantize_activation takes the block maximum with a maximum that
 * ignores NaN: a NaN input does not poison its block's scale (torch's amax would propagate it); the NaN element
 * itself goes through the hardware's saturating e4m3 conversion.  Inputs are expected to be finite.  A zero keeps
 * its sign through both quantisers (the activation quantiser and the FP8-output epilogue): -0.0, and a negative
 * whose quotient rounds to zero, become e4m3 0x80 as in the torch quantiser.
 */

/* Kernel launches issued by this library in this process so far. */
int64_t gu_launch_count(void);

/*
 * Time limit of every bounded device-side wait on the current device, in nanoseconds (default 2 s; 0 restores
 * the default).  A wait that runs out records (wait id, block) for gu_last_status, the kernel's roles skip the
 * rest of their device work and the launch returns; nothing traps.  The reference has no counterpart: its
 * cluster wait spins without bound (variants/cute_fused_v1/blockwise_gemm_fused.py:85-91).  Synchronous copy of
 * one word to the device; set it while no launch of this library is in flight.
 */
int gu_set_wait_limit_ns(uint64_t ns);

/*
 * Self-test of the bounded-wait protocol: launches one CTA whose only wait is on a barrier nothing ever arrives
 * on.  It returns after the wait limit (lower it first with gu_set_wait_limit_ns: the default is 2 s); afterwards
 * gu_last_status reports GU_ETIMEOUT with wait id 31, and the context stays usable.  Nothing traps or faults, no
 * copy or MMA is in flight.  No counterpart in the reference.
 */
int gu_wait_probe(void* stream);

/*
 * Cycle counters of the CTA-pair kernel's roles (what each role of the first CTA pair spent waiting for the
 * others, summed over the launches since the last clear).  Only a library built with -DGU_TRACE fills them;
 * the regular build returns 0 and writes nothing.  Copies up to `capacity` 64-bit words to `out` (layout:
 * [2 CTAs][16 slots] of summed cycles, then [2 CTAs][2 roles][64] time stamps of sixteen K blocks of the first
 * tile; all named in csrc/gateup_pair.cuh), returns the number of words written (at most 288) or a negative
 * code; `clear` != 0 zeroes the counters afterwards.  Synchronises the device.  Profiling aid with no
 * counterpart in the reference.
 */
int gu_trace_read(uint64_t* out, int capacity, int clear);

#ifdef __cplusplus
}
#endif
#endif /* GATEUP_H_ */
