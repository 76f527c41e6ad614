// torch bindings of the tcgen05 GEMM family.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kernels.h"

namespace {

using at::Tensor;

// One int32 error word per device, written by kernels whose bounded waits ran
// out.  Read (with a device sync) through device_status().
Tensor& status_word(int device) {
  static std::vector<Tensor> words(64);
  if (!words[device].defined()) {
    words[device] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  }
  return words[device];
}

int64_t device_status() {
  int dev = at::cuda::current_device();
  Tensor& w = status_word(dev);
  int64_t v = w.cpu().data_ptr<int>()[0];
  if (v != 0) w.zero_();
  return v;
}

Tensor gemm(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, int64_t act,
            bool a_mn, bool b_mn) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm: 2-D operands required");
  TORCH_CHECK(a.scalar_type() == b.scalar_type() &&
                  (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "gemm: bf16 or fp16 operands of the same type required");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "gemm: innermost dimension must be contiguous");
  c10::cuda::CUDAGuard guard(a.device());
  const int M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  const int K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  const int N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  const int Kb = static_cast<int>(b_mn ? b.size(0) : b.size(1));
  TORCH_CHECK(K == Kb, "gemm: contraction sizes differ: ", K, " vs ", Kb);
  Tensor c = at::empty({M, N}, a.options());
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == a.scalar_type() && bias->numel() == N && bias->is_contiguous(),
                "gemm: bias must be a contiguous [N] tensor of the operand dtype");
    bias_ptr = bias->data_ptr();
  }
  int rc = slapo::launch_gemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), bias_ptr, M, N, K,
                              static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)), N,
                              a_mn, b_mn, a.scalar_type() == at::kBFloat16, static_cast<int>(act),
                              status_word(a.get_device()).data_ptr<int>(),
                              at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "gemm: launch refused (code ", rc,
              "): sizes must be multiples of 8 and pointers 16-byte aligned");
  return c;
}

}  // namespace

int* slapo_status_ptr(int device) { return status_word(device).data_ptr<int>(); }

void register_gemm_ops(torch::Library& m) {
  m.def("gemm(Tensor a, Tensor b, Tensor? bias, int act, bool a_mn, bool b_mn) -> Tensor", &gemm);
  m.def("device_status() -> int", &device_status);
}
