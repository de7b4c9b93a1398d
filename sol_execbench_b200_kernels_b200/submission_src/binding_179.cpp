// Torch binding of the FP8 gate/up kernel for a SOL-ExecBench "cuda_cpp" submission of problem 179: the
// evaluator compiles the listed sources as one torch extension and calls run(*inputs, *outputs).  Same
// signature and checks as the reference's C++ variant (variants/cuda_cpp_v4/binding.cpp:18-81), without its
// fixed K and N; everything below the checks goes through the C ABI of gateup.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdint>
#include <map>
#include <mutex>
#include <utility>

#include "gateup.h"

namespace {

void check_cuda_contiguous(const torch::Tensor& t, const char* name, c10::ScalarType dtype, const char* dtype_name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", dtype_name);
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// Scratch of the small-M plan (stream-K hand-off flags and partial sums): one buffer per (device, stream),
// grown on demand and initialised once per allocation.  It carries no numbers from one call to the next:
// every call stamps the flags it reads with a fresh epoch.
torch::Tensor workspace_for(const torch::Tensor& like, cudaStream_t stream, size_t bytes) {
  static std::mutex mutex;
  static std::map<std::pair<int, cudaStream_t>, torch::Tensor> cache;
  std::lock_guard<std::mutex> lock(mutex);
  auto key = std::make_pair(static_cast<int>(like.get_device()), stream);
  auto it = cache.find(key);
  if (it == cache.end() || static_cast<size_t>(it->second.numel()) < bytes) {
    torch::Tensor ws = torch::empty({static_cast<int64_t>(bytes)}, like.options().dtype(torch::kUInt8));
    const int rc = gu_workspace_init(ws.data_ptr(), bytes, stream);
    TORCH_CHECK(rc == GU_OK, "gu_workspace_init: ", gu_error_string(rc));
    cache[key] = ws;
    return ws;
  }
  return it->second;
}

}  // namespace

void run(const torch::Tensor& x, const torch::Tensor& scale_x, const torch::Tensor& gate_proj_weight,
         const torch::Tensor& scale_gate, const torch::Tensor& up_proj_weight, const torch::Tensor& scale_up,
         torch::Tensor output) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
  c10::cuda::CUDAGuard guard(x.device());
  check_cuda_contiguous(x, "x", torch::kFloat8_e4m3fn, "float8_e4m3fn");
  check_cuda_contiguous(gate_proj_weight, "gate_proj_weight", torch::kFloat8_e4m3fn, "float8_e4m3fn");
  check_cuda_contiguous(up_proj_weight, "up_proj_weight", torch::kFloat8_e4m3fn, "float8_e4m3fn");
  check_cuda_contiguous(scale_x, "scale_x", torch::kFloat32, "float32");
  check_cuda_contiguous(scale_gate, "scale_gate", torch::kFloat32, "float32");
  check_cuda_contiguous(scale_up, "scale_up", torch::kFloat32, "float32");
  check_cuda_contiguous(output, "output", torch::kBFloat16, "bfloat16");
  TORCH_CHECK(x.dim() == 2 && gate_proj_weight.dim() == 2 && up_proj_weight.dim() == 2, "x and the weights must be 2-D");
  const int64_t m = x.size(0), k = x.size(1), n = gate_proj_weight.size(0);
  TORCH_CHECK(m >= 1 && k >= 128 && n >= 128 && k % 128 == 0 && n % 128 == 0,
              "need M >= 1 and K, N multiples of 128");
  TORCH_CHECK(gate_proj_weight.size(1) == k && up_proj_weight.size(0) == n && up_proj_weight.size(1) == k,
              "gate_proj_weight and up_proj_weight must have shape [N, K]");
  TORCH_CHECK(scale_x.sizes() == torch::IntArrayRef({m, k / 128}), "scale_x must have shape [M, K/128]");
  TORCH_CHECK(scale_gate.sizes() == torch::IntArrayRef({n / 128, k / 128}), "scale_gate must have shape [N/128, K/128]");
  TORCH_CHECK(scale_up.sizes() == torch::IntArrayRef({n / 128, k / 128}), "scale_up must have shape [N/128, K/128]");
  TORCH_CHECK(output.sizes() == torch::IntArrayRef({m, n}), "output must have shape [M, N]");
  const int device = x.get_device();
  TORCH_CHECK(scale_x.get_device() == device && gate_proj_weight.get_device() == device &&
                  scale_gate.get_device() == device && up_proj_weight.get_device() == device &&
                  scale_up.get_device() == device && output.get_device() == device,
              "all tensors must be on the same CUDA device");

  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device);
  gu_problem pr{};
  pr.x = x.data_ptr();
  pr.scale_x = scale_x.data_ptr<float>();
  pr.gate_w = gate_proj_weight.data_ptr();
  pr.scale_gate = scale_gate.data_ptr<float>();
  pr.up_w = up_proj_weight.data_ptr();
  pr.scale_up = scale_up.data_ptr<float>();
  pr.output = output.data_ptr();
  pr.m = m;
  pr.k = k;
  pr.n = n;
  pr.ld_output = n;
  pr.plan = GU_PLAN_AUTO;
  torch::Tensor ws;
  const size_t need = gu_workspace_bytes(m, k, n, GU_PLAN_AUTO);
  if (need != 0) {
    ws = workspace_for(x, stream, need);
    pr.workspace = ws.data_ptr();
    pr.workspace_bytes = static_cast<size_t>(ws.numel());
  }
  const int rc = gu_run(&pr, stream);
  TORCH_CHECK(rc == GU_OK, "gu_run: ", gu_error_string(rc));
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) { module.def("run", &run, "FP8 gate/up projection with SwiGLU (B200)"); }
