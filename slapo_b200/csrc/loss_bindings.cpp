// torch bindings of the cross-entropy and gradient-norm kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kernels.h"

namespace {

using at::Tensor;

int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return 0;
    case at::kHalf: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "slapo_b200: unsupported dtype ", t.scalar_type());
  }
}

void check_logits(const Tensor& logits, const Tensor& labels) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1,
              "logits must be a 2-D CUDA tensor with a contiguous last dimension");
  TORCH_CHECK(logits.size(1) % 8 == 0 && logits.stride(0) % 8 == 0,
              "vocabulary slice and row stride must be multiples of 8");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous() &&
                  labels.numel() == logits.size(0),
              "labels must be a contiguous int64 CUDA tensor with one entry per row");
}

// [rows, 3] fp32: (row max, sum exp(x - max), target logit or 0)
Tensor ce_stats(const Tensor& logits, const Tensor& labels, int64_t vocab_start,
                int64_t ignore_index) {
  check_logits(logits, labels);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor stats = at::empty({logits.size(0), 3}, logits.options().dtype(at::kFloat));
  slapo::launch_ce_stats(logits.data_ptr(), labels.data_ptr<int64_t>(), stats.data_ptr<float>(),
                         static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                         logits.stride(0), static_cast<int>(vocab_start), ignore_index,
                         dtype_code(logits), at::cuda::getCurrentCUDAStream().stream());
  return stats;
}

Tensor ce_grad(const Tensor& logits, const Tensor& labels, const Tensor& lse, const Tensor& coef,
               int64_t vocab_start, int64_t ignore_index) {
  check_logits(logits, labels);
  TORCH_CHECK(lse.scalar_type() == at::kFloat && coef.scalar_type() == at::kFloat &&
              lse.is_contiguous() && coef.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor grad = at::empty_strided(logits.sizes(), logits.strides(), logits.options());
  slapo::launch_ce_grad(logits.data_ptr(), labels.data_ptr<int64_t>(), lse.data_ptr<float>(),
                        coef.data_ptr<float>(), grad.data_ptr(), static_cast<int>(logits.size(0)),
                        static_cast<int>(logits.size(1)), logits.stride(0),
                        static_cast<int>(vocab_start), ignore_index, dtype_code(logits),
                        at::cuda::getCurrentCUDAStream().stream());
  return grad;
}

// out[0] = sum x^2 over mask == 0 (all of x without a mask), out[1] = over mask != 0
Tensor sq_norm(const Tensor& x, const c10::optional<Tensor>& mask) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.numel() % 8 == 0);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::zeros({2}, x.options().dtype(at::kFloat));
  const uint8_t* mp = nullptr;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->numel() == x.numel() && mask->element_size() == 1 && mask->is_contiguous());
    mp = static_cast<const uint8_t*>(mask->data_ptr());
  }
  slapo::launch_sq_norm(x.data_ptr(), mp, out.data_ptr<float>(), x.numel(), dtype_code(x),
                        at::cuda::getCurrentCUDAStream().stream());
  return out;
}

}  // namespace

void register_loss_ops(torch::Library& m) {
  m.def("ce_stats(Tensor logits, Tensor labels, int vocab_start, int ignore_index) -> Tensor",
        &ce_stats);
  m.def("ce_grad(Tensor logits, Tensor labels, Tensor lse, Tensor coef, int vocab_start, int ignore_index) -> Tensor",
        &ce_grad);
  m.def("sq_norm(Tensor x, Tensor? mask) -> Tensor", &sq_norm);
}
