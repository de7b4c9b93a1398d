/*
 * Plain C restatement of the FP8 gate/up projection + SwiGLU.  TEST INFRASTRUCTURE ONLY: built by
 * oracle/build_c.py into oracle/_build/ and loaded by the tests; nothing in the package links or calls it.
 *
 * It states every step on bits and scalars, with no tensor library underneath:
 *   - e4m3fn decode by table (1 sign, 4 exponent bits biased by 7, 3 mantissa bits; 0x7f / 0xff NaN);
 *   - per 128-wide K block the inner product in double (the products of two e4m3 values are exact and 128 of them
 *     sum exactly in 53 bits), rounded once to fp32 — what an exact-accumulating tensor core leaves;
 *   - acc += partial * (scale_x[m, j] * scale_w[n / 128, j]) as one fused multiply-add per block, blocks ascending:
 *     the promotion order of the reference's GEMM (variants/cute_fused_v1/blockwise_gemm_fused.py:1817-1823);
 *   - bf16 round-to-nearest-even by integer arithmetic after each GEMM, after SiLU and after the product, the
 *     three boundaries of kernels/179_fp8_mlp_gate_up_projection/kernel.py:165-171 and
 *     variants/cuda_cpp_v4/kernel.cu:250-260.
 * Sizes the loops finish in seconds only (M * N * K up to about 1e9).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float e4m3_table[256];
static int table_ready = 0;

static void build_table(void) {
  for (int c = 0; c < 256; ++c) {
    const int e = (c >> 3) & 0xF, m = c & 7;
    double v;
    if ((c & 0x7F) == 0x7F) {
      v = NAN;
    } else if (e == 0) {
      v = ldexp((double)m, -9);
    } else {
      v = ldexp((double)(8 + m), e - 10);
    }
    e4m3_table[c] = (float)((c & 0x80) ? -v : v);
  }
  table_ready = 1;
}

static uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* fp32 -> bf16 bits, round to nearest even (NaN stays NaN) */
static uint16_t bf16_bits(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float bf16_round(float f) { return bits_f32((uint32_t)bf16_bits(f) << 16); }

/* one fp32 GEMM element in the kernels' order */
static float blockwise_dot(const uint8_t* x_row, const float* sx_row, const uint8_t* w_row, const float* sw_row,
                           int64_t kb) {
  float acc = 0.0f;
  for (int64_t j = 0; j < kb; ++j) {
    double partial = 0.0;
    for (int t = 0; t < 128; ++t) partial += (double)e4m3_table[x_row[j * 128 + t]] * (double)e4m3_table[w_row[j * 128 + t]];
    acc = fmaf((float)partial, sx_row[j] * sw_row[j], acc);
  }
  return acc;
}

/*
 * x [M, K], gate_w / up_w [N, K]: e4m3fn bytes; scale_x [M, K/128], scale_gate / scale_up [N/128, K/128]: fp32;
 * out [M, N]: bf16 bits.  Returns 0, or -1 when K or N is not a multiple of 128.
 */
int gateup_oracle_c(const uint8_t* x, const float* scale_x, const uint8_t* gate_w, const float* scale_gate,
                    const uint8_t* up_w, const float* scale_up, uint16_t* out, int64_t m, int64_t k, int64_t n) {
  if (k % 128 != 0 || n % 128 != 0 || m < 0) return -1;
  if (!table_ready) build_table();
  const int64_t kb = k / 128;
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t c = 0; c < n; ++c) {
      const float g32 = blockwise_dot(x + i * k, scale_x + i * kb, gate_w + c * k, scale_gate + (c / 128) * kb, kb);
      const float u32 = blockwise_dot(x + i * k, scale_x + i * kb, up_w + c * k, scale_up + (c / 128) * kb, kb);
      const float g = bf16_round(g32);
      const float u = bf16_round(u32);
      const float act = bf16_round(g / (1.0f + expf(-g)));
      out[i * n + c] = bf16_bits(act * u);
    }
  }
  return 0;
}

/* the single block-scaled GEMM (down projection): c [M, N] bf16 bits */
int gemm_oracle_c(const uint8_t* a, const float* scale_a, const uint8_t* b, const float* scale_b, uint16_t* c_out,
                  int64_t m, int64_t k, int64_t n) {
  if (k % 128 != 0 || n % 128 != 0 || m < 0) return -1;
  if (!table_ready) build_table();
  const int64_t kb = k / 128;
  for (int64_t i = 0; i < m; ++i)
    for (int64_t c = 0; c < n; ++c)
      c_out[i * n + c] = bf16_bits(blockwise_dot(a + i * k, scale_a + i * kb, b + c * k, scale_b + (c / 128) * kb, kb));
  return 0;
}
