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
// product and the exact-residual correction (q0 = x*r; e = fma(-q0, s, x); q = fma(e, r, q0)), and the
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
};

// Blocks in flight per half-warp: enough 16-byte loads outstanding to cover HBM latency at full bandwidth
template <typename T>
__host__ __device__ constexpr int quant_unroll() { return sizeof(T) == 2 ? 8 : 4; }

// kPitched = false: rows are contiguous (ld_x == K), block b starts at element 128 * b and no division is needed.
template <typename T, bool kPitched>
__global__ void __launch_bounds__(kQuantThreads)
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
      const float s = fmaxf(amax, 1e-12f) / 448.0f;
      const float r = __frcp_rn(s);
      auto quot = [&](float a) {
        const float q0 = a * r;
        return fmaf(fmaf(-q0, s, a), r, q0);
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
            const float a = quot(v[4 * w + 2 * i]);
            const float c = quot(v[4 * w + 2 * i + 1]);
            const __nv_fp8x2_storage_t pair = __nv_cvt_float2_to_fp8x2(make_float2(a, c), __NV_SATFINITE, __NV_E4M3);
            word |= static_cast<uint32_t>(pair) << (16 * i);
          }
          packed[w] = word;
        }
        __stcs(reinterpret_cast<uint2*>(q + static_cast<long long>(bb) * 128 + sub * 8), make_uint2(packed[0], packed[1]));
        if (sub == 0) scale[bb] = s;
      }
    }
  }
}

}  // namespace gu
