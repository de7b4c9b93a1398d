/*
 * libsideops.so — C ABI of the two HBM-bound operators that live beside the FP8 gate/up path in the
 * reference repository: problem 038 (per-head RMSNorm of the Flux query / key tensors) and the
 * depthwise-convolution tail of problem 029 (Mamba conv1d with gating).  sm_100a only.
 *
 * Conventions (as in gateup.h): plain device pointers on the current device, no allocation inside the
 * library, launches on the stream that is passed in, 0 or a negative code is returned, argument errors are
 * detected before any CUDA call.
 */
#ifndef SIDEOPS_H_
#define SIDEOPS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SO_OK 0
#define SO_EINVAL_NULL -1  /* a required pointer is null */
#define SO_EINVAL_SHAPE -2 /* a size is outside the contract */
#define SO_EINVAL_ALIGN -3 /* a pointer is not 16-byte aligned */
#define SO_ECUDA -4        /* the launch failed */
#define SO_EDEVICE -5      /* the current device is not a compute capability 10.x GPU */
#define SO_ETIMEOUT -6     /* so_last_status: a bounded device-side wait of an earlier launch ran out */
#define SO_EBOUNDS -7      /* so_last_status, range-checked debug build only: an index or coordinate was out of range */

int so_version(void);
const char* so_error_string(int code);

/*
 * Per-head RMSNorm of query and key in one launch:
 *   out[t, h, :] = in[t, h, :] * rsqrt(mean(in[t, h, :]^2) + eps) * weight[h, :]
 * for both tensors, fp32 throughout.  query, key, query_norm, key_norm: [tokens, heads, 128] contiguous
 * (any leading batch dimensions flattened into `tokens`); weight_q, weight_k: [heads, 128].
 * Replaces `run` of kernels/038_flux_multi_head_rmsnorm_qk/binding.cpp:26-64 and
 * `launch_flux_rmsnorm_qk` of kernel.cu:229-268, which fix heads = 48; here heads is any positive count,
 * the head width stays 128 (one warp-wide 16-byte access per row).
 */
int so_rmsnorm_qk(const float* query, const float* key, const float* weight_q, const float* weight_k, float eps,
                  float* query_norm, float* key_norm, int64_t tokens, int heads, void* stream);

/*
 * Tail of the Mamba mixer after the input projection (kernels/029_mamba_conv1d_with_gating/kernel.cu:162-258,
 * launched from kernel.cu:316-347 and binding.cpp:95-101).  All tensors bf16.
 *   projected       [batch, sequence, projected_width]; channels [0, channels) of the last axis are the
 *                   convolution input (the rest, the gate, is not touched)
 *   attention_mask  [batch, sequence], values 0 or 1
 *   conv_weight     [channels, 4]   (a [channels, 1, 4] depthwise kernel), conv_bias [channels]
 *   output          [batch, channels, sequence]  — transposed relative to the input
 * Per (b, c, l):  x[j] = bf16(projected[b, l-3+j, c] * mask[b, l-3+j]) (0 before the sequence start);
 *   conv = bf16(((x0*w0 + x1*w1) + x2*w2) + x3*w3 + bias) accumulated in fp32 in that order;
 *   sig = bf16(1 / (1 + exp(-conv)));  act = bf16(conv * sig);  output = act where mask[b, l] >= 0.5, else 0.
 * The reference fixes channels = 16384, projected_width = 32768; here channels is any multiple of 64 and
 * projected_width any multiple of 8 that is >= channels.
 */
int so_mamba_conv1d_tail(const void* projected, const void* attention_mask, const void* conv_weight,
                         const void* conv_bias, void* output, int64_t batch, int64_t sequence, int64_t channels,
                         int64_t projected_width, void* stream);

/*
 * Input projection of the Mamba mixer: projected[m, n] = bf16(hidden[m, k] . weight[n, k]^T + bias[n]); all tensors
 * bf16 row-major and contiguous, fp32 accumulation, the bias added in fp32 before the one rounding.  One launch of
 * a persistent tcgen05 (kind::f16) kernel: CTA pairs on 256 x 256 tiles for m > 128, lone CTAs on 128 x 256 tiles
 * otherwise.  Replaces `launch_sm100_cutlass_projection` of kernels/029_mamba_conv1d_with_gating/kernel.cu:274-312
 * (a CUTLASS builder GEMM with a row-broadcast bias, kernel.cu:36-160), which fixes k = 8192 and n = 32768 and needs
 * m to be B x L of a [B, L, 8192] tensor; here m >= 0 and k, n are any multiples of 8 (rows are 16-byte aligned).
 * Every device-side wait of the kernel is bounded; so_last_status reports one that ran out.
 */
int so_mamba_in_proj(const void* hidden, const void* weight, const void* bias, void* projected, int64_t m, int64_t k,
                     int64_t n, void* stream);

/*
 * Synchronises the device and returns SO_OK, or SO_ETIMEOUT if a bounded wait inside so_mamba_in_proj ran out since
 * the status was last cleared (`detail`: wait id << 24 | block), or SO_EBOUNDS (range-checked build); `clear` != 0
 * resets it.
 */
int so_last_status(int* detail, int clear);

/*
 * 1 in the range-checked debug build (-DGU_BOUNDS=1: the projection kernel tests every computed TMA coordinate, bias
 * index and ring stage against its extent, records the first violation — so_last_status then returns SO_EBOUNDS with
 * detail = site << 16 | block — and skips the access), 0 in the regular library.
 */
int so_is_range_checked_build(void);

/* Time limit of the device-side waits in nanoseconds (0 restores the default of 2 s).  Synchronises the device. */
int so_set_wait_limit_ns(uint64_t ns);

/* Number of kernel launches issued by this library in this process. */
int64_t so_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SIDEOPS_H_ */
