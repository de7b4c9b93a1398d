// SOL-ExecBench problem 029 as a "cuda_cpp" submission.  Six bf16 inputs in, (output_hidden_states, gate) out, as
// the reference's entry point has it (kernels/029_mamba_conv1d_with_gating/binding.cpp:31-104).  Two calls into the
// C ABI of sideops.h on torch's current stream: the input projection (bf16 GEMM with the bias in its epilogue) and
// everything after it; `gate` is a transposed view of the projection's upper half, never copied.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <array>
#include <tuple>
#include <utility>

#include "sideops.h"

namespace {

using Named = std::pair<const torch::Tensor*, const char*>;

template <size_t N>
void require_dense_bf16_on(const std::array<Named, N>& operands, int device) {
  for (const Named& operand : operands) {
    const torch::Tensor& t = *operand.first;
    TORCH_CHECK(t.is_cuda() && t.get_device() == device, operand.second, ": expected a CUDA tensor on device ", device);
    TORCH_CHECK(t.scalar_type() == torch::kBFloat16, operand.second, ": expected bfloat16, got ", t.scalar_type());
    TORCH_CHECK(t.is_contiguous(), operand.second, ": expected a contiguous tensor");
  }
}

}  // namespace

std::tuple<torch::Tensor, torch::Tensor> run(const torch::Tensor& hidden_states, const torch::Tensor& attention_mask,
                                             const torch::Tensor& in_proj_weight, const torch::Tensor& in_proj_bias,
                                             const torch::Tensor& conv1d_weight, const torch::Tensor& conv1d_bias) {
  TORCH_CHECK(hidden_states.is_cuda(), "hidden_states: expected a CUDA tensor");
  const int device = hidden_states.get_device();
  c10::cuda::CUDAGuard guard(hidden_states.device());
  require_dense_bf16_on<6>({{{&hidden_states, "hidden_states"}, {&attention_mask, "attention_mask"},
                             {&in_proj_weight, "in_proj_weight"}, {&in_proj_bias, "in_proj_bias"},
                             {&conv1d_weight, "conv1d_weight"}, {&conv1d_bias, "conv1d_bias"}}}, device);

  // sizes: B x L tokens of width H; the projection makes 2 C columns, the lower C of them are convolved
  TORCH_CHECK(hidden_states.dim() == 3, "hidden_states: expected [B, L, H]");
  const int64_t B = hidden_states.size(0), L = hidden_states.size(1), H = hidden_states.size(2);
  TORCH_CHECK(in_proj_weight.dim() == 2 && in_proj_weight.size(1) == H, "in_proj_weight: expected [2 C, ", H, "]");
  const int64_t two_c = in_proj_weight.size(0);
  TORCH_CHECK(two_c % 128 == 0, "in_proj_weight: 2 C must be a multiple of 128, got ", two_c);
  const int64_t C = two_c / 2;
  TORCH_CHECK(attention_mask.dim() == 2 && attention_mask.size(0) == B && attention_mask.size(1) == L,
              "attention_mask: expected [", B, ", ", L, "]");
  TORCH_CHECK(in_proj_bias.dim() == 1 && in_proj_bias.size(0) == two_c, "in_proj_bias: expected [", two_c, "]");
  TORCH_CHECK(conv1d_weight.dim() == 3 && conv1d_weight.size(0) == C && conv1d_weight.size(1) == 1 &&
                  conv1d_weight.size(2) == 4,
              "conv1d_weight: expected [", C, ", 1, 4]");
  TORCH_CHECK(conv1d_bias.dim() == 1 && conv1d_bias.size(0) == C, "conv1d_bias: expected [", C, "]");

  TORCH_CHECK(H % 8 == 0 && H >= 8, "hidden_states: H must be a multiple of 8, got ", H);
  torch::Tensor projection = torch::empty({B, L, two_c}, hidden_states.options());
  if (B > 0 && L > 0) {
    const int status = so_mamba_in_proj(hidden_states.data_ptr(), in_proj_weight.data_ptr(), in_proj_bias.data_ptr(),
                                        projection.data_ptr(), B * L, H, two_c,
                                        at::cuda::getCurrentCUDAStream(device).stream());
    TORCH_CHECK(status == SO_OK, "so_mamba_in_proj failed: ", so_error_string(status));
  }
  torch::Tensor gate = projection.narrow(/*dim=*/2, /*start=*/C, /*length=*/C).transpose(1, 2);
  torch::Tensor mixed = torch::empty({B, C, L}, hidden_states.options());
  if (B > 0 && L > 0) {
    const int status = so_mamba_conv1d_tail(projection.data_ptr(), attention_mask.data_ptr(), conv1d_weight.data_ptr(),
                                            conv1d_bias.data_ptr(), mixed.data_ptr(), B, L, C, two_c,
                                            at::cuda::getCurrentCUDAStream(device).stream());
    TORCH_CHECK(status == SO_OK, "so_mamba_conv1d_tail failed: ", so_error_string(status));
  }
  return {mixed, gate};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def("run", &run, "Mamba projection + conv1d tail (libsideops)"); }
