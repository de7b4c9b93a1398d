// Torch binding of the Mamba conv1d tail for a SOL-ExecBench "cuda_cpp" submission of problem 029.  Same
// six-argument signature and (output_hidden_states, gate) return as the reference's binding
// (kernels/029_mamba_conv1d_with_gating/binding.cpp:31-104): the input projection is a plain bf16 GEMM + bias
// and goes to the vendor library through at::linear; `gate` is the transposed view of its upper half; the tail
// goes through the C ABI of sideops.h.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/ops/linear.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <tuple>

#include "sideops.h"

namespace {
void check_bf16(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must have bfloat16 dtype");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
}  // namespace

std::tuple<torch::Tensor, torch::Tensor> run(const torch::Tensor& hidden_states, const torch::Tensor& attention_mask,
                                             const torch::Tensor& in_proj_weight, const torch::Tensor& in_proj_bias,
                                             const torch::Tensor& conv1d_weight, const torch::Tensor& conv1d_bias) {
  c10::cuda::CUDAGuard guard(hidden_states.device());
  check_bf16(hidden_states, "hidden_states");
  check_bf16(attention_mask, "attention_mask");
  check_bf16(in_proj_weight, "in_proj_weight");
  check_bf16(in_proj_bias, "in_proj_bias");
  check_bf16(conv1d_weight, "conv1d_weight");
  check_bf16(conv1d_bias, "conv1d_bias");
  TORCH_CHECK(hidden_states.dim() == 3, "hidden_states must have shape [B, L, H]");
  const int64_t batch = hidden_states.size(0), sequence = hidden_states.size(1), hidden = hidden_states.size(2);
  TORCH_CHECK(in_proj_weight.dim() == 2 && in_proj_weight.size(1) == hidden && in_proj_weight.size(0) % 2 == 0,
              "in_proj_weight must have shape [2 C, H]");
  const int64_t projected_width = in_proj_weight.size(0), channels = projected_width / 2;
  TORCH_CHECK(channels % 64 == 0, "the intermediate size must be a multiple of 64");
  TORCH_CHECK(attention_mask.sizes() == torch::IntArrayRef({batch, sequence}), "attention_mask must have shape [B, L]");
  TORCH_CHECK(in_proj_bias.sizes() == torch::IntArrayRef({projected_width}), "in_proj_bias must have shape [2 C]");
  TORCH_CHECK(conv1d_weight.sizes() == torch::IntArrayRef({channels, 1, 4}), "conv1d_weight must have shape [C, 1, 4]");
  TORCH_CHECK(conv1d_bias.sizes() == torch::IntArrayRef({channels}), "conv1d_bias must have shape [C]");
  const int device = hidden_states.get_device();
  TORCH_CHECK(attention_mask.get_device() == device && in_proj_weight.get_device() == device &&
                  in_proj_bias.get_device() == device && conv1d_weight.get_device() == device &&
                  conv1d_bias.get_device() == device,
              "all tensors must be on the same CUDA device");

  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device);
  torch::Tensor projected = at::linear(hidden_states, in_proj_weight, in_proj_bias);
  torch::Tensor gate = projected.slice(/*dim=*/2, channels, projected_width).transpose(1, 2);
  torch::Tensor output = torch::empty({batch, channels, sequence}, hidden_states.options());
  if (batch != 0 && sequence != 0) {
    const int rc = so_mamba_conv1d_tail(projected.data_ptr(), attention_mask.data_ptr(), conv1d_weight.data_ptr(),
                                        conv1d_bias.data_ptr(), output.data_ptr(), batch, sequence, channels,
                                        projected_width, stream);
    TORCH_CHECK(rc == SO_OK, "so_mamba_conv1d_tail: ", so_error_string(rc));
  }
  return std::make_tuple(output, gate);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) { module.def("run", &run, "Mamba projection, causal conv1d and SiLU"); }
