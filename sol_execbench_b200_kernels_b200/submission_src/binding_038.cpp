// SOL-ExecBench problem 038 as a "cuda_cpp" submission: the evaluator builds the listed sources into one torch
// extension and calls run(*inputs, *outputs).  Argument order and destination passing follow the reference's
// entry point (kernels/038_flux_multi_head_rmsnorm_qk/binding.cpp:26-64); the work is one call into the C ABI of
// sideops.h, on torch's current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <array>
#include <utility>

#include "sideops.h"

namespace {

using Named = std::pair<const torch::Tensor*, const char*>;

// every operand of this problem is a dense fp32 tensor on one GPU
template <size_t N>
void require_dense_f32_on(const std::array<Named, N>& operands, int device) {
  for (const Named& operand : operands) {
    const torch::Tensor& t = *operand.first;
    TORCH_CHECK(t.is_cuda() && t.get_device() == device, operand.second, ": expected a CUDA tensor on device ", device);
    TORCH_CHECK(t.scalar_type() == torch::kFloat32, operand.second, ": expected float32, got ", t.scalar_type());
    TORCH_CHECK(t.is_contiguous(), operand.second, ": expected a contiguous tensor");
  }
}

}  // namespace

void run(const torch::Tensor& query, const torch::Tensor& key, const torch::Tensor& weight_q,
         const torch::Tensor& weight_k, double eps, torch::Tensor query_norm, torch::Tensor key_norm) {
  TORCH_CHECK(query.is_cuda(), "query: expected a CUDA tensor");
  const int device = query.get_device();
  c10::cuda::CUDAGuard guard(query.device());
  require_dense_f32_on<6>({{{&query, "query"}, {&key, "key"}, {&weight_q, "weight_q"}, {&weight_k, "weight_k"},
                            {&query_norm, "query_norm"}, {&key_norm, "key_norm"}}}, device);

  const int64_t rank = query.dim();
  TORCH_CHECK(rank >= 3, "query: expected [..., heads, 128], got ", rank, " dimensions");
  const int64_t heads = query.size(rank - 2);
  const int64_t width = query.size(rank - 1);
  TORCH_CHECK(width == 128, "query: the head width must be 128, got ", width);
  TORCH_CHECK(key.sizes() == query.sizes(), "key: shape differs from query");
  TORCH_CHECK(query_norm.sizes() == query.sizes(), "query_norm: shape differs from query");
  TORCH_CHECK(key_norm.sizes() == query.sizes(), "key_norm: shape differs from query");
  for (const Named& w : {Named{&weight_q, "weight_q"}, Named{&weight_k, "weight_k"}}) {
    TORCH_CHECK(w.first->dim() == 2 && w.first->size(0) == heads && w.first->size(1) == width, w.second,
                ": expected shape [", heads, ", ", width, "]");
  }

  const int64_t tokens = query.numel() / (heads * width);
  if (tokens == 0) return;  // nothing to normalise
  const int status = so_rmsnorm_qk(query.data_ptr<float>(), key.data_ptr<float>(), weight_q.data_ptr<float>(),
                                   weight_k.data_ptr<float>(), static_cast<float>(eps),
                                   query_norm.data_ptr<float>(), key_norm.data_ptr<float>(), tokens,
                                   static_cast<int>(heads), at::cuda::getCurrentCUDAStream(device).stream());
  TORCH_CHECK(status == SO_OK, "so_rmsnorm_qk failed: ", so_error_string(status));
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def("run", &run, "per-head RMSNorm of query and key (libsideops)"); }
