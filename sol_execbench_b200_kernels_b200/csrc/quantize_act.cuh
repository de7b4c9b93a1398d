// Activation quantiser: the step in front of the gate/up projection.
//
//   x[M, K] (bf16 or fp32)  ->  q[M, K] e4m3  +  scale[M, K/128] fp32,   scale = amax(1x128 block) / 448
//
// The reference receives its activations already quantised (kernels/179_fp8_mlp_gate_up_projection/
// kernel.py:356-357); this produces them on the GPU in the layout its entry point takes.  Pure streaming:
// every element is read once and written once, so the kernel is HBM-bound.  A lane owns eight consecutive
// elements (one 16- or 32-byte load), sixteen lanes own one 128-wide block, so a warp instruction covers
// two blocks; the block maximum is a four-step shuffle reduction inside the half-warp.  The quotient
// x / scale is the correctly rounded one: one correctly rounded reciprocal per block, then per element a
// product and the exact-residual correction (q0 = x*r; e = fma(-q0, s, x); q = fma(e, r, q0); two elements per
// instruction with the packed fp32 forms), and the
// conversion rounds to nearest even with saturation, so the bits equal those of
// `clamp(x / scale, -448, 448).to(float8_e4m3fn)` in PyTorch at a fifth of the instructions of eight divisions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gu {

constexpr int kQuantThreads = 256;

// Eight consecutive elements, kept as loaded (packed) while further loads are in flight.
template <typename T>
struct Raw8;
template <>
struct Raw8<__nv_bfloat16> {
  uint4 w;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { w = __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void zero() { w = make_uint4(0, 0, 0, 0); }
  // fp32 values and the largest magnitude (the maximum of bf16 values is exact in bf16: two elements per instruction)
  __device__ __forceinline__ float unpack(float (&v)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
    __nv_bfloat162 m2 = __habs2(h[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i > 0) m2 = __hmax2(m2, __habs2(h[i]));
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
    const float2 mf = __bfloat1622float2(m2);
    return fmaxf(mf.x, mf.y);
  }
  // the sign bits of elements 4w .. 4w+3 at bits 7, 15, 23, 31 (the high byte of each bf16, one byte permute)
  __device__ __forceinline__ uint32_t signs(int word) const {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&w);
    return __byte_perm(p[2 * word], p[2 * word + 1], 0x7531) & 0x80808080u;
  }
};
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldcs(reinterpret_cast<const float4*>(p));
    b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ float unpack(float (&v)[8]) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
  }
  // the sign bits of elements 4w .. 4w+3 at bits 7, 15, 23, 31 (the top byte of each float)
  __device__ __forceinline__ uint32_t signs(int word) const {
    const float4& f = word ? b : a;
    const uint32_t lo = __byte_perm(__float_as_uint(f.x), __float_as_uint(f.y), 0x0073);  // bytes: x.b3, y.b3, -, -
    const uint32_t hi = __byte_perm(__float_as_uint(f.z), __float_as_uint(f.w), 0x0073);
    return __byte_perm(lo, hi, 0x5410) & 0x80808080u;
  }
};

// a / 448, correctly rounded, without the division sequence: product with the rounded reciprocal, then the
// exact-residual correction (the same scheme as the per-element quotient).  Equal to the IEEE quotient for every
// fp32 input from 1e-12 up (checked on the CPU: all bf16-valued inputs, 10^8 random fp32 inputs).
__device__ __forceinline__ float div_by_448(float a) {
  constexpr float kInv448 = 0.0022321429569274187f;  // RN(1 / 448) = 0x3b124925
  const float q0 = a * kInv448;
  return fmaf(fmaf(-q0, 448.0f, a), kInv448, q0);
}

// 1 / s for a normal s whose reciprocal is normal (here 2e-15 <= s < 2^126): hardware approximation plus one
// residual step, in place of the general routine with its special-case branch.
__device__ __forceinline__ float reciprocal_normal(float s) {
  float r0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(s));
  return fmaf(fmaf(-s, r0, 1.0f), r0, r0);
}

// Blocks in flight per half-warp: enough 16-byte loads outstanding to cover HBM latency at full bandwidth
template <typename T>
__host__ __device__ constexpr int quant_unroll() { return 4; }
// Resident CTAs the compiler is asked to leave room for: measured on a B200 (bf16 input, 16384 x 7168, µs per launch,
// unroll x CTAs per SM): 4x6 61.3, 6x5 62.6, 8x4 63.1, 4x8 64.7, 12x4 67.2, 8x5 (spills) 67.8.
template <typename T>
__host__ __device__ constexpr int quant_min_ctas() { return sizeof(T) == 2 ? 6 : 1; }

// kPitched = false: rows are contiguous (ld_x == K), block b starts at element 128 * b and no division is needed.
template <typename T, bool kPitched>
__global__ void __launch_bounds__(kQuantThreads, quant_min_ctas<T>())
quantize_act_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, uint32_t blocks,
                    long long ld_x, uint32_t kb) {
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15;                 // position inside the half-warp: elements 8*sub .. 8*sub+7 of the block
  constexpr int kQuantUnroll = quant_unroll<T>();
  const uint32_t half_warps = gridDim.x * (kQuantThreads / 16);
  // the host keeps blocks + kQuantUnroll * half_warps below 2^32
  for (uint32_t b = blockIdx.x * (kQuantThreads / 16) + (threadIdx.x >> 4); b < blocks; b += half_warps * kQuantUnroll) {
    Raw8<T> raw[kQuantUnroll];
    bool live[kQuantUnroll];
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      const uint32_t bb = b + u * half_warps;
      live[u] = bb < blocks;
      if (live[u]) {
        if constexpr (kPitched) {
          const uint32_t row = bb / kb;
          const uint32_t j = bb - row * kb;
          raw[u].load(x + row * ld_x + static_cast<long long>(j) * 128 + sub * 8);
        } else {
          raw[u].load(x + static_cast<long long>(bb) * 128 + sub * 8);
        }
      } else {
        raw[u].zero();
      }
    }
#pragma unroll
    for (int u = 0; u < kQuantUnroll; ++u) {
      float v[8];
      float amax = raw[u].unpack(v);
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float s = div_by_448(fmaxf(amax, 1e-12f));
      const float r = reciprocal_normal(s);
      // two quotients per instruction with the packed fp32 forms
      const float2 r2 = make_float2(r, r), ns2 = make_float2(-s, -s);
      auto quot2 = [&](float a, float c) {
        const float2 x2 = make_float2(a, c);
        const float2 q0 = __fmul2_rn(x2, r2);
        return __ffma2_rn(__ffma2_rn(q0, ns2, x2), r2, q0);
      };
      if (live[u]) {
        const uint32_t bb = b + u * half_warps;
        uint32_t packed[2];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t word = 0;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            // |x| <= amax, so |x / s| <= 448 up to one rounding; the saturating conversion does the clamp
            const float2 ac = quot2(v[4 * w + 2 * i], v[4 * w + 2 * i + 1]);
            const __nv_fp8x2_storage_t pair = __nv_cvt_float2_to_fp8x2(ac, __NV_SATFINITE, __NV_E4M3);
            word |= static_cast<uint32_t>(pair) << (16 * i);
          }
          // (the residual step turns a quotient of -0 into +0; the source's sign bits put the sign of such a zero back:
          // a quotient never has the other sign, so the OR changes nothing else)
          word |= raw[u].signs(w);
          packed[w] = word;
        }
        __stcs(reinterpret_cast<uint2*>(q + static_cast<long long>(bb) * 128 + sub * 8), make_uint2(packed[0], packed[1]));
        if (sub == 0) scale[bb] = s;
      }
    }
  }
}

}  // namespace gu
