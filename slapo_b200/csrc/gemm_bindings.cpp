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

// fp32 scratch of the split-K pair GEMM (one slice per split; contents do not matter), one per
// device, grown on demand.  All GEMMs of a device run on one stream at a time.
Tensor& split_scratch(int device, int64_t floats) {
  static std::vector<Tensor> s(64);
  if (!s[device].defined() || s[device].numel() < floats)
    s[device] = at::empty({floats}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device));
  return s[device];
}

// impl: 0 = pick (CTA-pair kernel when the problem has at least one pair tile, else the
// single-CTA kernel), 1 = single-CTA kernel, 2 = CTA-pair kernel or fail.
// split_k: allow several CTA pairs per output tile (weight gradients).
// the word itself (device tensor), for callers that copy it out asynchronously
Tensor device_status_tensor() { return status_word(at::cuda::current_device()); }

Tensor gemm_out(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, int64_t act,
                bool a_mn, bool b_mn, const c10::optional<Tensor>& out,
                const c10::optional<Tensor>& pre_act, int64_t impl, bool split_k) {
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
  Tensor c;
  if (out.has_value() && out->defined()) {
    c = *out;
    TORCH_CHECK(c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1 &&
                    c.scalar_type() == a.scalar_type(),
                "gemm: `out` must be an [M, N] tensor of the operand dtype with contiguous rows");
  } else {
    c = at::empty({M, N}, a.options());
  }
  void* c2 = nullptr;
  if (pre_act.has_value() && pre_act->defined()) {
    TORCH_CHECK(pre_act->sizes() == c.sizes() && pre_act->strides() == c.strides() &&
                    pre_act->scalar_type() == c.scalar_type(),
                "gemm: `pre_act` must match the output's shape, strides and dtype");
    c2 = pre_act->data_ptr();
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == a.scalar_type() && bias->numel() == N && bias->is_contiguous(),
                "gemm: bias must be a contiguous [N] tensor of the operand dtype");
    bias_ptr = bias->data_ptr();
  }
  const int dev = a.get_device();
  const bool bf16 = a.scalar_type() == at::kBFloat16;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int rc = 5;
  if (impl != 1) {
    float* ws = nullptr;
    const int splits = split_k ? slapo::gemm2_splits(M, N, K, N > 128 ? 256 : 128) : 1;
    if (splits > 1) ws = split_scratch(dev, static_cast<int64_t>(splits) * M * N).data_ptr<float>();
    rc = slapo::launch_gemm2(a.data_ptr(), b.data_ptr(), c.data_ptr(), c2, bias_ptr, M, N, K,
                             static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)),
                             static_cast<int>(c.stride(0)), a_mn, b_mn, bf16,
                             static_cast<int>(act), ws,
                             status_word(dev).data_ptr<int>(), stream);
    TORCH_CHECK(impl != 2 || rc == 0, "gemm: the CTA-pair kernel refused the launch (code ", rc, ")");
  }
  if (rc == 5) {
    TORCH_CHECK(c2 == nullptr, "gemm: `pre_act` needs a problem of at least one 256 x 128 tile");
    rc = slapo::launch_gemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), bias_ptr, M, N, K,
                            static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)),
                            static_cast<int>(c.stride(0)), a_mn, b_mn, bf16, static_cast<int>(act),
                            status_word(dev).data_ptr<int>(), stream);
  }
  TORCH_CHECK(rc == 0, "gemm: launch refused (code ", rc,
              "): sizes must be multiples of 8 and pointers 16-byte aligned");
  return c;
}

Tensor gemm(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, int64_t act,
            bool a_mn, bool b_mn) {
  return gemm_out(a, b, bias, act, a_mn, b_mn, c10::nullopt, c10::nullopt, 0, false);
}

}  // namespace

int* slapo_status_ptr(int device) { return status_word(device).data_ptr<int>(); }

void register_gemm_ops(torch::Library& m) {
  m.def("gemm(Tensor a, Tensor b, Tensor? bias, int act, bool a_mn, bool b_mn) -> Tensor", &gemm);
  m.def("gemm_out(Tensor a, Tensor b, Tensor? bias, int act, bool a_mn, bool b_mn, Tensor? out, "
        "Tensor? pre_act, int impl, bool split_k) -> Tensor", &gemm_out);
  m.def("gemm2_splits(int M, int N, int K) -> int", [](int64_t M, int64_t N, int64_t K) -> int64_t {
    return slapo::gemm2_splits(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                               N > 128 ? 256 : 128);
  });
  m.def("device_status() -> int", &device_status);
  m.def("device_status_tensor() -> Tensor", &device_status_tensor);
}
