// Torch binding of the per-head RMSNorm kernel for a SOL-ExecBench "cuda_cpp" submission of problem 038.
// Same seven-argument, destination-passing signature and checks as the reference's binding
// (kernels/038_flux_multi_head_rmsnorm_qk/binding.cpp:26-64); the launch goes through the C ABI of sideops.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "sideops.h"

namespace {
void check_f32(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, " must have float32 dtype");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
}  // namespace

void run(const torch::Tensor& query, const torch::Tensor& key, const torch::Tensor& weight_q,
         const torch::Tensor& weight_k, double eps, torch::Tensor query_norm, torch::Tensor key_norm) {
  c10::cuda::CUDAGuard guard(query.device());
  check_f32(query, "query");
  check_f32(key, "key");
  check_f32(weight_q, "weight_q");
  check_f32(weight_k, "weight_k");
  check_f32(query_norm, "query_norm");
  check_f32(key_norm, "key_norm");
  TORCH_CHECK(query.dim() >= 3, "query must be [..., heads, 128]");
  TORCH_CHECK(query.sizes() == key.sizes(), "query and key shapes must match");
  const int64_t heads = query.size(-2);
  TORCH_CHECK(query.size(-1) == 128, "query and key must have heads of width 128");
  TORCH_CHECK(weight_q.sizes() == torch::IntArrayRef({heads, 128}), "weight_q must have shape [heads, 128]");
  TORCH_CHECK(weight_k.sizes() == torch::IntArrayRef({heads, 128}), "weight_k must have shape [heads, 128]");
  TORCH_CHECK(query_norm.sizes() == query.sizes(), "query_norm shape must match query");
  TORCH_CHECK(key_norm.sizes() == key.sizes(), "key_norm shape must match key");
  const int device = query.get_device();
  TORCH_CHECK(key.get_device() == device && weight_q.get_device() == device && weight_k.get_device() == device &&
                  query_norm.get_device() == device && key_norm.get_device() == device,
              "all tensors must use the same CUDA device");
  const int64_t tokens = query.numel() / (heads * 128);
  if (tokens == 0) return;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device);
  const int rc = so_rmsnorm_qk(query.data_ptr<float>(), key.data_ptr<float>(), weight_q.data_ptr<float>(),
                               weight_k.data_ptr<float>(), static_cast<float>(eps), query_norm.data_ptr<float>(),
                               key_norm.data_ptr<float>(), tokens, static_cast<int>(heads), stream);
  TORCH_CHECK(rc == SO_OK, "so_rmsnorm_qk: ", so_error_string(rc));
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) { module.def("run", &run, "Flux query/key per-head RMSNorm"); }
