// libsideops.so: the operators that sit beside the FP8 gate/up path in the reference repository — per-head
// RMSNorm of the Flux query / key tensors (problem 038) and both halves of the Mamba mixer's front end (problem 029):
// the bf16 input projection with bias (a tcgen05 GEMM, proj_gemm.cuh) and the depthwise convolution + SiLU tail.
// sm_100a only; the C ABI is include/sideops.h.
#include "../../include/sideops.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "proj_gemm.cuh"

namespace so {

std::atomic<long long> g_launches{0};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------------------------------------------
// Per-head RMSNorm of query and key (problem 038).
//
// A row is one (token, head) vector of 128 fp32 = 512 bytes = one float4 per lane.  A warp owns
// kRowsPerWarp consecutive rows and issues all of their loads before the first reduction, so that every
// thread keeps 64 bytes in flight; blockIdx.y selects the tensor (0 query, 1 key).  Algorithmic traffic:
// 2 tensors x (read + write) x 512 bytes per row; the [heads, 128] weights stay in L1/L2.
// ------------------------------------------------------------------------------------------------------------
constexpr int kNormRowsPerWarp = 4;
constexpr int kNormWarps = 8;
constexpr int kNormRowsPerBlock = kNormRowsPerWarp * kNormWarps;

__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_qk_kernel(const float4* __restrict__ query, const float4* __restrict__ key,
                  const float4* __restrict__ weight_q, const float4* __restrict__ weight_k, float eps,
                  float4* __restrict__ query_norm, float4* __restrict__ key_norm, long long rows, int heads) {
  const bool is_key = blockIdx.y != 0;
  const float4* __restrict__ in = is_key ? key : query;
  const float4* __restrict__ weight = is_key ? weight_k : weight_q;
  float4* __restrict__ out = is_key ? key_norm : query_norm;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long row0 = (static_cast<long long>(blockIdx.x) * kNormWarps + warp) * kNormRowsPerWarp;

  float4 v[kNormRowsPerWarp];
  float sum[kNormRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kNormRowsPerWarp; ++i) {
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + i < rows) v[i] = __ldg(in + (row0 + i) * 32 + lane);
  }
  // the weight rows are fetched before the reduction so that their latency hides behind it
  float4 wv[kNormRowsPerWarp];
  {
    int head = static_cast<int>(row0 % heads);
#pragma unroll
    for (int i = 0; i < kNormRowsPerWarp; ++i) {
      wv[i] = __ldg(weight + head * 32 + lane);
      if (++head == heads) head = 0;
    }
  }
#pragma unroll
  for (int i = 0; i < kNormRowsPerWarp; ++i)
    sum[i] = fmaf(v[i].w, v[i].w, fmaf(v[i].z, v[i].z, fmaf(v[i].y, v[i].y, v[i].x * v[i].x)));
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
#pragma unroll
    for (int i = 0; i < kNormRowsPerWarp; ++i) sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], offset);
  }
#pragma unroll
  for (int i = 0; i < kNormRowsPerWarp; ++i) {
    if (row0 + i < rows) {
      const float4 w = wv[i];
      const float s = rsqrtf(fmaf(sum[i], 1.0f / 128.0f, eps));
      float4 r;
      r.x = (v[i].x * s) * w.x;
      r.y = (v[i].y * s) * w.y;
      r.z = (v[i].z * s) * w.z;
      r.w = (v[i].w * s) * w.w;
      out[(row0 + i) * 32 + lane] = r;  // default policy: the consumer of the normalised tensors reads them next
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Mamba conv1d tail (problem 029): mask -> depthwise causal conv (4 taps) + bias -> SiLU -> mask, with the
// [sequence, channel] -> [channel, sequence] transposition done through shared memory.
//
// A CTA owns 64 channels x 128 positions.  Load phase: 131 rows (3 rows of history) of 128 contiguous bytes,
// 16 bytes per thread, pre-masked.  Compute phase: a lane owns a channel PAIR (one 32-bit shared-memory word
// per row, so a warp reads 128 contiguous bytes), a warp owns 16 positions and slides the 4-tap window along
// them; the fp32 arithmetic is done on (channel, channel+1) pairs with the packed f32x2 instructions.  Two
// positions of one channel are packed into one word of the transposed output tile (pitch 66 words).  Store
// phase: 256 contiguous bytes per warp instruction (8 bytes per lane) when the sequence length is a multiple
// of 4, 128 when it is even, single elements when it is odd.  Algorithmic traffic: 2 bytes read + 2 bytes written per
// (token, channel).
//
// The sigmoid costs 1.25 special-function operations per element instead of 2 (see sigmoid_2x2): for arguments
// >= -20 it is 1 / (1 + 2^(-x log2 e)) with ONE reciprocal of the product of the four denominators of a 2 x 2
// block; a run that holds an argument below -20 takes the wide-range form sigmoid_wide, which keeps full relative
// accuracy in the negative tail.
// ------------------------------------------------------------------------------------------------------------
constexpr int kConvChannels = 64;
constexpr int kConvPositions = 128;
constexpr int kConvTaps = 4;
constexpr int kConvRows = kConvPositions + kConvTaps - 1;  // 131
constexpr int kConvThreads = 256;
constexpr int kConvOutPitch = kConvPositions / 2 + 2;  // words; even, so that rows stay 8-byte aligned for the 64-bit reads of the store phase
constexpr int kConvRun = kConvPositions / (kConvThreads / 32);  // positions per warp = 16

__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t float2_to_bf16x2(float2 v) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(v.y), "f"(v.x));
  return r;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// bf16(a * m) for both halves of a packed word; the fp32 product of two bf16 values is exact, so this is the
// single rounding of the eager masked multiply
__device__ __forceinline__ uint32_t mask_mul_bf16x2(uint32_t a, uint32_t m2) { return mul_bf16x2(a, m2); }

// convolution + bias for one position of a channel pair, rounded to bf16 (packed)
__device__ __forceinline__ uint32_t conv_pair(float2 x0, float2 x1, float2 x2, float2 x3, const float2 (&w)[4],
                                              float2 bias) {
  float2 acc = __fmul2_rn(x0, w[0]);
  acc = __ffma2_rn(x1, w[1], acc);
  acc = __ffma2_rn(x2, w[2], acc);
  acc = __ffma2_rn(x3, w[3], acc);
  acc = __fadd2_rn(acc, bias);
  return float2_to_bf16x2(acc);
}

// sigmoid of one value in full relative accuracy at any magnitude: e = 2^(-|x| log2 e) with log2 e split into a
// 16-bit head (its product with an 8-bit bf16 significand is exact in fp32) and a tail applied as a first-order
// factor; 1/(1+e) for x >= 0, e/(1+e) for x < 0
__device__ __noinline__ float sigmoid_wide(float x) {
  constexpr float kLog2eHead = 1.44268798828125f;      // 0x3fb8aa00
  constexpr float kLog2eTailLn2 = 4.888495152129525e-06f;  // (log2 e - head) * ln 2
  const float a = fabsf(x);
  const float e0 = ex2_approx(-a * kLog2eHead);
  const float e = fmaf(e0, -a * kLog2eTailLn2, e0);
  const float r = rcp_approx(1.0f + e);
  return x < 0.f ? e * r : r;
}

// bf16(sigmoid) of the four bf16 values in two packed words (channel pair at two positions), all four
// arguments >= -20: sigmoid = 1 / (1 + 2^(-x log2 e)) directly; each denominator is below 2^30, so the product of
// the four stays finite and ONE reciprocal of it serves all four (products of the other three give each quotient
// back): 1.25 special-function operations per element instead of 2.
__device__ __forceinline__ void sigmoid_2x2(uint32_t ca, uint32_t cb, uint32_t& sa, uint32_t& sb) {
  constexpr float kNegLog2e = -1.4426950408889634f;
  const float2 scale = make_float2(kNegLog2e, kNegLog2e);
  const float2 ta = __fmul2_rn(bf16x2_to_float2(ca), scale);
  const float2 tb = __fmul2_rn(bf16x2_to_float2(cb), scale);
  const float2 one = make_float2(1.f, 1.f);
  const float2 ya = __fadd2_rn(make_float2(ex2_approx(ta.x), ex2_approx(ta.y)), one);
  const float2 yb = __fadd2_rn(make_float2(ex2_approx(tb.x), ex2_approx(tb.y)), one);
  const float2 pab = __fmul2_rn(ya, yb);        // (ya.x*yb.x, ya.y*yb.y)
  const float inv = rcp_approx(pab.x * pab.y);  // 1 / (all four)
  const float2 rab = make_float2(inv * pab.y, inv * pab.x);  // 1/(ya.x*yb.x), 1/(ya.y*yb.y)
  sa = float2_to_bf16x2(__fmul2_rn(rab, yb));   // 1/ya
  sb = float2_to_bf16x2(__fmul2_rn(rab, ya));   // 1/yb
}

__global__ void __launch_bounds__(kConvThreads)  // 48 registers: 5 CTAs per SM; forcing 6 (40 registers) measured 7 % slower
mamba_conv1d_tail_kernel(const __nv_bfloat16* __restrict__ projected, const __nv_bfloat16* __restrict__ mask,
                         const __nv_bfloat16* __restrict__ conv_weight, const __nv_bfloat16* __restrict__ conv_bias,
                         __nv_bfloat16* __restrict__ output, int sequence, int channels, long long width) {
  __shared__ __align__(16) uint32_t s_in[kConvRows * (kConvChannels / 2)];  // [row][channel pair]
  __shared__ __align__(8) uint32_t s_out[kConvChannels * kConvOutPitch];                 // [channel][position pair]
  __shared__ uint32_t s_keep[kConvPositions / 2];  // per position pair: 0xffff in the half of a kept position

  const int tid = threadIdx.x;
  const int batch = blockIdx.z;
  const int c0 = blockIdx.x * kConvChannels;
  const int l0 = blockIdx.y * kConvPositions;
  const long long token0 = static_cast<long long>(batch) * sequence;
  const uint16_t* mask_bits = reinterpret_cast<const uint16_t*>(mask) + token0;

  // ---- load phase: 131 rows x 8 chunks of 16 bytes.  Thread t owns chunk t % 8 of rows t / 8 + 32 i, so its
  // addresses advance by a constant; all of its global loads are issued before the first use ----
  constexpr int kLoadsPerThread = (kConvRows + 31) / 32;  // 5; the last round has 3 rows
  const int l_first = l0 + (tid >> 3) - (kConvTaps - 1);
  uint4 raw[kLoadsPerThread];
  uint32_t m2[kLoadsPerThread];
  {
    const uint4* src = reinterpret_cast<const uint4*>(projected + token0 * width + c0) + (tid & 7);
    const long long row_pitch = width >> 3;  // 16-byte words per token row
    long long off = static_cast<long long>(l_first) * row_pitch;
#pragma unroll
    for (int i = 0; i < kLoadsPerThread; ++i) {
      const int l = l_first + 32 * i;
      raw[i] = make_uint4(0u, 0u, 0u, 0u);
      m2[i] = 0u;
      if ((i < kLoadsPerThread - 1 || tid < 8 * (kConvRows - 32 * (kLoadsPerThread - 1))) && l >= 0 && l < sequence) {
        raw[i] = __ldcs(src + off);
        const uint32_t mb = __ldg(mask_bits + l);
        m2[i] = mb | (mb << 16);
      }
      off += 32 * row_pitch;
    }
  }
  if (tid < kConvPositions / 2) {
    // the reference keeps an output only where the mask is at least one half (bf16 bits 0x3f00 .. 0x7f80)
    uint32_t keep = 0u;
    const int l = l0 + 2 * tid;
    if (l < sequence && __ldg(mask_bits + l) - 0x3f00u <= 0x4080u) keep |= 0x0000ffffu;
    if (l + 1 < sequence && __ldg(mask_bits + l + 1) - 0x3f00u <= 0x4080u) keep |= 0xffff0000u;
    s_keep[tid] = keep;
  }
#pragma unroll
  for (int i = 0; i < kLoadsPerThread; ++i) {
    if (i < kLoadsPerThread - 1 || tid < 8 * (kConvRows - 32 * (kLoadsPerThread - 1))) {
      uint4 v = raw[i];
      if (m2[i] != 0x3f803f80u) {  // a mask of exactly 1 leaves the values as they are
        v.x = mask_mul_bf16x2(v.x, m2[i]);
        v.y = mask_mul_bf16x2(v.y, m2[i]);
        v.z = mask_mul_bf16x2(v.z, m2[i]);
        v.w = mask_mul_bf16x2(v.w, m2[i]);
      }
      reinterpret_cast<uint4*>(s_in)[tid + i * kConvThreads] = v;
    }
  }

  // ---- per-thread constants: taps and bias of this lane's channel pair ----
  const int lane = tid & 31;
  const int warp = tid >> 5;
  float2 w[4], bias;
  {
    const int c = c0 + 2 * lane;
    const uint4 wq = __ldg(reinterpret_cast<const uint4*>(conv_weight + static_cast<long long>(c) * kConvTaps));
    const float2 wa01 = bf16x2_to_float2(wq.x), wa23 = bf16x2_to_float2(wq.y);  // channel c, taps 0..3
    const float2 wb01 = bf16x2_to_float2(wq.z), wb23 = bf16x2_to_float2(wq.w);  // channel c + 1
    w[0] = make_float2(wa01.x, wb01.x);
    w[1] = make_float2(wa01.y, wb01.y);
    w[2] = make_float2(wa23.x, wb23.x);
    w[3] = make_float2(wa23.y, wb23.y);
    bias = bf16x2_to_float2(__ldg(reinterpret_cast<const uint32_t*>(conv_bias + c)));
  }
  __syncthreads();

  // ---- compute phase: this warp's 16 positions in two halves.  Per half: all convolutions (sliding window),
  // one test whether every result allows the short sigmoid, then sigmoid and product two positions at a time ----
  {
    constexpr int kHalf = kConvRun / 2;
    const int p0 = warp * kConvRun;
    const uint32_t* col = s_in + p0 * 32 + lane;
    // tile row of channel c is (c & 1) * 32 + (c >> 1): the lanes of a warp store to consecutive rows (a 2-way
    // bank conflict at the even pitch, cheaper than a second pass of 32-bit global stores)
    uint32_t* dst_a = s_out + lane * kConvOutPitch + (p0 >> 1);
    uint32_t* dst_b = dst_a + 32 * kConvOutPitch;
    const uint32_t* keep = s_keep + (p0 >> 1);
    float2 x0 = bf16x2_to_float2(col[0 * 32]);
    float2 x1 = bf16x2_to_float2(col[1 * 32]);
    float2 x2 = bf16x2_to_float2(col[2 * 32]);
#pragma unroll
    for (int h = 0; h < kConvRun; h += kHalf) {
      uint32_t conv[kHalf];
#pragma unroll
      for (int j = 0; j < kHalf; ++j) {
        const float2 x3 = bf16x2_to_float2(col[(h + j + 3) * 32]);
        conv[j] = conv_pair(x0, x1, x2, x3, w, bias);  // position p0 + h + j, channels (c, c + 1)
        x0 = x1;
        x1 = x2;
        x2 = x3;
      }
      __nv_bfloat162 lowest = *reinterpret_cast<const __nv_bfloat162*>(&conv[0]);
#pragma unroll
      for (int j = 1; j < kHalf; ++j) lowest = __hmin2(lowest, *reinterpret_cast<const __nv_bfloat162*>(&conv[j]));
      if (__hbge2(lowest, __floats2bfloat162_rn(-20.f, -20.f))) {
#pragma unroll
        for (int j = 0; j < kHalf; j += 2) {
          uint32_t sa, sb;
          sigmoid_2x2(conv[j], conv[j + 1], sa, sb);
          const uint32_t ra = mul_bf16x2(conv[j], sa);
          const uint32_t rb = mul_bf16x2(conv[j + 1], sb);
          const uint32_t k2 = keep[(h + j) >> 1];
          dst_a[(h + j) >> 1] = __byte_perm(ra, rb, 0x5410) & k2;  // channel c:     positions p, p + 1
          dst_b[(h + j) >> 1] = __byte_perm(ra, rb, 0x7632) & k2;  // channel c + 1: positions p, p + 1
        }
      } else {  // some result below -20 (or a NaN): the wide-range sigmoid for this half, rare
#pragma unroll  // unrolled although cold: a run-time index would move conv[] to local memory for both branches
        for (int j = 0; j < kHalf; j += 2) {
          const float2 xa = bf16x2_to_float2(conv[j]);
          const float2 xb = bf16x2_to_float2(conv[j + 1]);
          const uint32_t sa = float2_to_bf16x2(make_float2(sigmoid_wide(xa.x), sigmoid_wide(xa.y)));
          const uint32_t sb = float2_to_bf16x2(make_float2(sigmoid_wide(xb.x), sigmoid_wide(xb.y)));
          const uint32_t ra = mul_bf16x2(conv[j], sa);
          const uint32_t rb = mul_bf16x2(conv[j + 1], sb);
          const uint32_t k2 = keep[(h + j) >> 1];
          dst_a[(h + j) >> 1] = __byte_perm(ra, rb, 0x5410) & k2;
          dst_b[(h + j) >> 1] = __byte_perm(ra, rb, 0x7632) & k2;
        }
      }
    }
  }
  __syncthreads();

  // ---- store phase: rows of the transposed tile, whole 256- or 128-byte runs per warp instruction ----
  const long long out_row0 = (static_cast<long long>(batch) * channels + c0) * sequence + l0;
  if ((sequence & 3) == 0) {
    // thread t owns positions 4 (t % 32) .. +3 of tile rows t / 32 + 8 i: rows 0..31 even channels, 32..63 odd
    const int pw = tid & 31;
    const int r0 = tid >> 5;
    if (l0 + 4 * pw < sequence) {
      const long long row_words = sequence >> 2;  // 8-byte words per output row
      uint2* dst = reinterpret_cast<uint2*>(output + out_row0) + 2 * r0 * row_words + pw;
      const uint32_t* src = s_out + r0 * kConvOutPitch + 2 * pw;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t* a = src + 8 * i * kConvOutPitch;
        const uint32_t* b = src + (32 + 8 * i) * kConvOutPitch;
        __stcs(dst, *reinterpret_cast<const uint2*>(a));
        __stcs(dst + row_words, *reinterpret_cast<const uint2*>(b));
        dst += 16 * row_words;
      }
    }
  } else if ((sequence & 1) == 0) {
    // thread t owns word t % 64 of tile rows t / 64 + 4 i: rows 0..31 are the even channels, 32..63 the odd ones
    const int wd = tid & 63;
    const int r0 = tid >> 6;
    if (l0 + 2 * wd < sequence) {
      const long long row_words = sequence >> 1;
      uint32_t* dst = reinterpret_cast<uint32_t*>(output + out_row0) + 2 * r0 * row_words + wd;
      const uint32_t* src = s_out + r0 * kConvOutPitch + wd;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __stcs(dst, src[4 * i * kConvOutPitch]);                      // channel 2 (r0 + 4 i)
        __stcs(dst + row_words, src[(32 + 4 * i) * kConvOutPitch]);   // channel 2 (r0 + 4 i) + 1
        dst += 8 * row_words;
      }
    }
  } else {  // odd row pitch: rows are only 2-byte aligned
    const uint16_t* s_out16 = reinterpret_cast<const uint16_t*>(s_out);
    uint16_t* out16 = reinterpret_cast<uint16_t*>(output);
    for (int idx = tid; idx < kConvChannels * kConvPositions; idx += kConvThreads) {
      const int r = idx >> 7;
      const int c = ((r & 31) << 1) | (r >> 5);
      const int p = idx & 127;
      if (l0 + p < sequence) out16[out_row0 + static_cast<long long>(c) * sequence + p] = s_out16[r * (2 * kConvOutPitch) + p];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Host side of the input projection: tensor maps, per-device set-up, launch.
// ------------------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// resolved through the runtime, so the library has no link-time dependency on the driver library
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 row-major [rows, cols], box [box_rows, 64 columns = 128 bytes], 128-byte swizzle; out-of-range reads are zero
int bf16_map(CUtensorMap* out, const void* ptr, uint64_t cols, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return SO_ECUDA;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SO_OK : SO_ECUDA;
}

struct ProjDevice {
  bool ready = false;
  int sm_count = 0;
  int pair_clusters = 0;  // two-CTA clusters of the pair kernel that are resident at once
};
std::mutex g_proj_mutex;
ProjDevice g_proj_dev[64];

int proj_device(ProjDevice** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SO_ECUDA;
  std::lock_guard<std::mutex> lock(g_proj_mutex);
  ProjDevice& d = g_proj_dev[dev];
  if (!d.ready) {
    int major = 0;
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return SO_ECUDA;
    if (major != 10) return SO_EDEVICE;
    if (cudaFuncSetAttribute(proj_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             PjCfg<true>::smem_bytes) != cudaSuccess ||
        cudaFuncSetAttribute(proj_gemm_lone_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             PjCfg<false>::smem_bytes) != cudaSuccess) {
      cudaGetLastError();
      return SO_ECUDA;
    }
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * static_cast<unsigned>(d.sm_count), 1, 1);
    cfg.blockDim = dim3(kPjThreads, 1, 1);
    cfg.dynamicSmemBytes = PjCfg<true>::smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, proj_gemm_pair_kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    d.pair_clusters = clusters;
    d.ready = true;
  }
  *out = &d;
  return SO_OK;
}

int launch_projection(const void* hidden, const void* weight, const void* bias, void* projected, int64_t m, int64_t k,
                      int64_t n, cudaStream_t stream) {
  ProjDevice* dev = nullptr;
  int rc = proj_device(&dev);
  if (rc != SO_OK) return rc;
  const bool pair = m > kPjTileM && dev->pair_clusters >= 1;
  CUtensorMap tm_a, tm_w, tm_o;
  if ((rc = bf16_map(&tm_a, hidden, k, m, kPjTileM)) != SO_OK) return rc;
  if ((rc = bf16_map(&tm_w, weight, k, n, pair ? PjCfg<true>::b_rows : PjCfg<false>::b_rows)) != SO_OK) return rc;
  if ((rc = bf16_map(&tm_o, projected, n, m, kPjTileM)) != SO_OK) return rc;
  ProjParams p;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.kb = static_cast<int>((k + kPjBlockK - 1) / kPjBlockK);
  const int rows_per_tile = pair ? PjCfg<true>::rows_per_tile : PjCfg<false>::rows_per_tile;
  p.m_tiles = static_cast<int>((m + rows_per_tile - 1) / rows_per_tile);
  p.n_tiles = static_cast<int>((n + kPjTileN - 1) / kPjTileN);
  const int64_t tiles = int64_t(p.m_tiles) * p.n_tiles;
  if (tiles * p.kb >= (1ll << 31)) return SO_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  // Raster: the tiles that run at the same time form a block of about 8 row tiles x (resident tiles / 8) column
  // tiles and walk K together, so a K block of `hidden` or `weight` is fetched from HBM once per block, not per tile.
  p.group_m = p.m_tiles < 8 ? p.m_tiles : 8;
  if (pair) {
    const int clusters = p.num_tiles < dev->pair_clusters ? p.num_tiles : dev->pair_clusters;
    proj_gemm_pair_kernel<<<2 * clusters, kPjThreads, PjCfg<true>::smem_bytes, stream>>>(tm_a, tm_w, tm_o, p);
  } else {
    const int ctas = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
    proj_gemm_lone_kernel<<<ctas, kPjThreads, PjCfg<false>::smem_bytes, stream>>>(tm_a, tm_w, tm_o, p);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? SO_OK : SO_ECUDA;
}

}  // namespace so

extern "C" {

int so_version(void) { return 1; }

const char* so_error_string(int code) {
  switch (code) {
    case SO_OK: return "ok";
    case SO_EINVAL_NULL: return "a required pointer is null";
    case SO_EINVAL_SHAPE: return "a size is outside the contract";
    case SO_EINVAL_ALIGN: return "a pointer is not 16-byte aligned";
    case SO_ECUDA: return "the CUDA launch failed";
    case SO_EDEVICE: return "the current device is not a compute capability 10.x GPU";
    case SO_ETIMEOUT: return "a device-side wait of an earlier launch ran out; its output is not valid";
    case SO_EBOUNDS: return "the range-checked debug build found an index or coordinate outside its extent";
    default: return "unknown error code";
  }
}

int64_t so_launch_count(void) { return so::g_launches.load(std::memory_order_relaxed); }

int so_rmsnorm_qk(const float* query, const float* key, const float* weight_q, const float* weight_k, float eps,
                  float* query_norm, float* key_norm, int64_t tokens, int heads, void* stream) {
  if (!query || !key || !weight_q || !weight_k || !query_norm || !key_norm) return SO_EINVAL_NULL;
  if (tokens < 0 || heads < 1 || tokens > (1ll << 40) / heads) return SO_EINVAL_SHAPE;
  if (!so::aligned16(query) || !so::aligned16(key) || !so::aligned16(weight_q) || !so::aligned16(weight_k) ||
      !so::aligned16(query_norm) || !so::aligned16(key_norm))
    return SO_EINVAL_ALIGN;
  if (tokens == 0) return SO_OK;
  const long long rows = tokens * heads;
  const long long blocks = (rows + so::kNormRowsPerBlock - 1) / so::kNormRowsPerBlock;
  if (blocks > 0x7fffffffll) return SO_EINVAL_SHAPE;
  const dim3 grid(static_cast<unsigned>(blocks), 2);
  so::rmsnorm_qk_kernel<<<grid, so::kNormWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(query), reinterpret_cast<const float4*>(key),
      reinterpret_cast<const float4*>(weight_q), reinterpret_cast<const float4*>(weight_k), eps,
      reinterpret_cast<float4*>(query_norm), reinterpret_cast<float4*>(key_norm), rows, heads);
  so::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? SO_OK : SO_ECUDA;
}

int so_mamba_conv1d_tail(const void* projected, const void* attention_mask, const void* conv_weight,
                         const void* conv_bias, void* output, int64_t batch, int64_t sequence, int64_t channels,
                         int64_t projected_width, void* stream) {
  if (!projected || !attention_mask || !conv_weight || !conv_bias || !output) return SO_EINVAL_NULL;
  if (batch < 0 || sequence < 0 || channels < so::kConvChannels || channels % so::kConvChannels != 0 ||
      projected_width < channels || projected_width % 8 != 0 || batch > 65535 || sequence > (1ll << 30) ||
      channels > (1ll << 30))
    return SO_EINVAL_SHAPE;
  if (!so::aligned16(projected) || !so::aligned16(conv_weight) || (reinterpret_cast<uintptr_t>(conv_bias) & 3u) ||
      (reinterpret_cast<uintptr_t>(attention_mask) & 1u) || !so::aligned16(output))
    return SO_EINVAL_ALIGN;
  if (batch == 0 || sequence == 0) return SO_OK;
  const long long seq_tiles = (sequence + so::kConvPositions - 1) / so::kConvPositions;
  if (seq_tiles > 65535) return SO_EINVAL_SHAPE;
  const dim3 grid(static_cast<unsigned>(channels / so::kConvChannels), static_cast<unsigned>(seq_tiles),
                  static_cast<unsigned>(batch));
  so::mamba_conv1d_tail_kernel<<<grid, so::kConvThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(projected), static_cast<const __nv_bfloat16*>(attention_mask),
      static_cast<const __nv_bfloat16*>(conv_weight), static_cast<const __nv_bfloat16*>(conv_bias),
      static_cast<__nv_bfloat16*>(output), static_cast<int>(sequence), static_cast<int>(channels), projected_width);
  so::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? SO_OK : SO_ECUDA;
}

int so_mamba_in_proj(const void* hidden, const void* weight, const void* bias, void* projected, int64_t m, int64_t k,
                     int64_t n, void* stream) {
  if (!hidden || !weight || !bias || !projected) return SO_EINVAL_NULL;
  if (m < 0 || k < 8 || n < 8 || k % 8 != 0 || n % 8 != 0 || m >= (1ll << 31) || k >= (1ll << 31) || n >= (1ll << 31))
    return SO_EINVAL_SHAPE;
  if (!so::aligned16(hidden) || !so::aligned16(weight) || !so::aligned16(bias) || !so::aligned16(projected))
    return SO_EINVAL_ALIGN;
  if (m == 0) return SO_OK;
  return so::launch_projection(hidden, weight, bias, projected, m, k, n, static_cast<cudaStream_t>(stream));
}

int so_last_status(int* detail, int clear) {
  unsigned int host[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return SO_ECUDA;
  if (cudaMemcpyFromSymbol(host, gu::g_status, sizeof(host)) != cudaSuccess) return SO_ECUDA;
  if (detail) *detail = static_cast<int>(host[1]);
  if (clear && host[0] != 0) {
    const unsigned int zero[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(gu::g_status, zero, sizeof(zero)) != cudaSuccess) return SO_ECUDA;
  }
  if (host[0] == 0) return SO_OK;
  return host[0] == gu::kStatusBounds ? SO_EBOUNDS : SO_ETIMEOUT;
}

int so_is_range_checked_build(void) {
#ifdef GU_BOUNDS
  return 1;
#else
  return 0;
#endif
}

int so_set_wait_limit_ns(uint64_t ns) {
  const unsigned long long v = ns ? ns : 2000000000ull;
  if (cudaDeviceSynchronize() != cudaSuccess) return SO_ECUDA;
  return cudaMemcpyToSymbol(gu::g_wait_limit_ns, &v, sizeof(v)) == cudaSuccess ? SO_OK : SO_ECUDA;
}

}  // extern "C"
