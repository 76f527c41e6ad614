// torch.ops.slapo_b200.* : tensor-level entry points of the sm_100a kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kernels.h"

namespace {

using at::Tensor;
using c10::optional;

int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return 0;
    case at::kHalf: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "slapo_b200: unsupported dtype ", t.scalar_type());
  }
}

const void* opt_ptr(const optional<Tensor>& t) {
  return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr;
}

void check_cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// Reserve `increment` Philox offsets on the current device's default
// generator.  Returns [seed|seed_ptr, offset|offset_ptr, intragraph, captured]
// as a CPU int64 tensor: valid both eagerly and under CUDA-graph capture (the
// pointers are stable, the generator refreshes what they point to per replay).
Tensor philox_reserve(int64_t increment) {
  auto gen = at::get_generator_or_default<at::CUDAGeneratorImpl>(
      c10::nullopt, at::cuda::detail::getDefaultCUDAGenerator());
  at::PhiloxCudaState st;
  {
    std::lock_guard<std::mutex> lock(gen->mutex_);
    st = gen->philox_cuda_state(static_cast<uint64_t>((increment + 3) / 4 * 4));
  }
  Tensor out = at::empty({4}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
  int64_t* o = out.data_ptr<int64_t>();
  if (st.captured_) {
    o[0] = reinterpret_cast<int64_t>(st.seed_.ptr);
    o[1] = reinterpret_cast<int64_t>(st.offset_.ptr);
  } else {
    o[0] = static_cast<int64_t>(st.seed_.val);
    o[1] = static_cast<int64_t>(st.offset_.val);
  }
  o[2] = static_cast<int64_t>(st.offset_intragraph_);
  o[3] = st.captured_ ? 1 : 0;
  return out;
}

slapo::PhiloxArgs unpack_rng(const optional<Tensor>& rng) {
  slapo::PhiloxArgs a{};
  if (!rng.has_value() || !rng->defined()) return a;
  TORCH_CHECK(rng->device().is_cpu() && rng->scalar_type() == at::kLong && rng->numel() == 4,
              "rng must be the CPU int64[4] tensor returned by philox_reserve");
  const int64_t* r = rng->data_ptr<int64_t>();
  a.captured = static_cast<int>(r[3]);
  a.offset_intragraph = static_cast<uint32_t>(r[2]);
  if (a.captured) {
    a.seed_ptr = reinterpret_cast<const int64_t*>(r[0]);
    a.offset_ptr = reinterpret_cast<const int64_t*>(r[1]);
  } else {
    a.seed = static_cast<uint64_t>(r[0]);
    a.offset = static_cast<uint64_t>(r[1]);
  }
  return a;
}

// ------------------------------------------------------------------------ //
Tensor bias_act_fwd(const Tensor& x, const optional<Tensor>& bias, int64_t act) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1);
  TORCH_CHECK(cols % 8 == 0, "last dimension must be a multiple of 8");
  Tensor y = at::empty_like(x);
  slapo::launch_bias_act_fwd(x.data_ptr(), opt_ptr(bias), y.data_ptr(), x.numel() / cols,
                             static_cast<int>(cols), static_cast<int>(act), dtype_code(x),
                             cur_stream());
  return y;
}

std::tuple<Tensor, Tensor> bias_act_bwd(const Tensor& dy, const Tensor& x,
                                        const optional<Tensor>& bias, int64_t act) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  Tensor dx = at::empty_like(x);
  Tensor dbias = at::empty({0}, x.options()), partial;
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) {
    dbias = at::empty_like(*bias);
    partial = at::empty({slapo::colsum_chunks(rows, cols), cols}, x.options().dtype(at::kFloat));
  }
  slapo::launch_bias_act_bwd(dy.data_ptr(), x.data_ptr(), opt_ptr(bias), dx.data_ptr(),
                             has_bias ? dbias.data_ptr() : nullptr,
                             has_bias ? partial.data_ptr<float>() : nullptr, rows, cols,
                             static_cast<int>(act), dtype_code(x), cur_stream());
  return {dx, dbias};
}

// dz = dy * act'(z), dbias = column sums of dz: the backward of an activation whose input z
// already contains the bias (the GEMM epilogue added it)
std::tuple<Tensor, Tensor> act_bwd_colsum(const Tensor& dy, const Tensor& z, int64_t act) {
  check_cuda_contig(dy, "dy");
  check_cuda_contig(z, "z");
  c10::cuda::CUDAGuard guard(z.device());
  const int cols = static_cast<int>(z.size(-1));
  const int rows = static_cast<int>(z.numel() / cols);
  TORCH_CHECK(cols % 8 == 0, "last dimension must be a multiple of 8");
  Tensor dz = at::empty_like(z);
  Tensor dbias = at::empty({cols}, z.options());
  Tensor partial = at::empty({slapo::colsum_chunks(rows, cols), cols}, z.options().dtype(at::kFloat));
  slapo::launch_bias_act_bwd(dy.data_ptr(), z.data_ptr(), nullptr, dz.data_ptr(), dbias.data_ptr(),
                             partial.data_ptr<float>(), rows, cols, static_cast<int>(act),
                             dtype_code(z), cur_stream());
  return {dz, dbias};
}

// column sums of a 2-D tensor with contiguous rows (row stride free)
Tensor colsum(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "colsum: 2-D CUDA tensor with contiguous rows");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0)), cols = static_cast<int>(x.size(1));
  TORCH_CHECK(cols % 8 == 0 && x.stride(0) % 8 == 0, "colsum: columns and row stride must be multiples of 8");
  Tensor out = at::empty({cols}, x.options());
  if (rows == 0) return out.zero_();
  Tensor partial = at::empty({slapo::colsum_chunks(rows, cols), cols}, x.options().dtype(at::kFloat));
  slapo::launch_colsum(x.data_ptr(), out.data_ptr(), partial.data_ptr<float>(), rows, cols,
                       x.stride(0), dtype_code(x), cur_stream());
  return out;
}

Tensor bias_dropout_add_fwd(const Tensor& x, const optional<Tensor>& bias,
                            const optional<Tensor>& residual, double p, const Tensor& rng) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1);
  TORCH_CHECK(cols % 8 == 0, "last dimension must be a multiple of 8");
  Tensor y = at::empty_like(x);
  slapo::launch_bias_dropout_add_fwd(x.data_ptr(), opt_ptr(bias), opt_ptr(residual), y.data_ptr(),
                                     x.numel() / cols, static_cast<int>(cols),
                                     static_cast<float>(p), unpack_rng(rng), dtype_code(x),
                                     cur_stream());
  return y;
}

std::tuple<Tensor, Tensor> bias_dropout_add_bwd(const Tensor& dy, double p, const Tensor& rng,
                                                bool want_dbias) {
  check_cuda_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(dy.device());
  const int cols = static_cast<int>(dy.size(-1));
  const int rows = static_cast<int>(dy.numel() / cols);
  Tensor dx = at::empty_like(dy);
  Tensor dbias = at::empty({0}, dy.options()), partial;
  if (want_dbias) {
    dbias = at::empty({cols}, dy.options());
    partial = at::empty({slapo::colsum_chunks(rows, cols), cols}, dy.options().dtype(at::kFloat));
  }
  slapo::launch_bias_dropout_add_bwd(dy.data_ptr(), dx.data_ptr(),
                                     want_dbias ? dbias.data_ptr() : nullptr,
                                     want_dbias ? partial.data_ptr<float>() : nullptr, rows, cols,
                                     static_cast<float>(p), unpack_rng(rng), dtype_code(dy),
                                     cur_stream());
  return {dx, dbias};
}

// ------------------------------------------------------------------------ //
std::tuple<Tensor, Tensor, Tensor> layer_norm_fwd(const Tensor& x, const Tensor& gamma,
                                                  const optional<Tensor>& beta, double eps,
                                                  bool rms) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  TORCH_CHECK(cols % 8 == 0 && cols <= 16384, "unsupported hidden size ", cols);
  Tensor y = at::empty_like(x);
  Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  slapo::launch_ln_fwd(x.data_ptr(), nullptr, nullptr, gamma.data_ptr(), opt_ptr(beta),
                       y.data_ptr(), nullptr, mean.data_ptr<float>(), rstd.data_ptr<float>(), rows,
                       cols, static_cast<float>(eps), 0.f, slapo::PhiloxArgs{}, rms ? 1 : 0,
                       dtype_code(x), cur_stream());
  return {y, mean, rstd};
}

std::tuple<Tensor, Tensor, Tensor> layer_norm_bwd(const Tensor& gy, const Tensor& x,
                                                  const Tensor& gamma, const Tensor& mean,
                                                  const Tensor& rstd, bool rms) {
  check_cuda_contig(gy, "gy");
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  Tensor dx = at::empty_like(x);
  Tensor dgamma = at::empty_like(gamma);
  Tensor dbeta = at::empty_like(gamma);
  Tensor partial = at::empty({slapo::ln_bwd_grid(rows, cols), 3, cols},
                             x.options().dtype(at::kFloat));
  slapo::launch_ln_bwd(gy.data_ptr(), nullptr, x.data_ptr(), gamma.data_ptr(),
                       mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(), nullptr,
                       dgamma.data_ptr(), dbeta.data_ptr(), nullptr, partial.data_ptr<float>(),
                       rows, cols, 0.f, slapo::PhiloxArgs{}, rms ? 1 : 0, dtype_code(x),
                       cur_stream());
  return {dx, dgamma, dbeta};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> dropout_add_ln_fwd(
    const Tensor& x, const optional<Tensor>& bias, const Tensor& residual, const Tensor& gamma,
    const optional<Tensor>& beta, double p, double eps, const optional<Tensor>& rng) {
  check_cuda_contig(x, "x");
  check_cuda_contig(residual, "residual");
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  TORCH_CHECK(cols % 8 == 0 && cols <= 16384, "unsupported hidden size ", cols);
  Tensor y = at::empty_like(x);
  Tensor z = at::empty_like(x);
  Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  slapo::launch_ln_fwd(x.data_ptr(), opt_ptr(bias), residual.data_ptr(), gamma.data_ptr(),
                       opt_ptr(beta), y.data_ptr(), z.data_ptr(), mean.data_ptr<float>(),
                       rstd.data_ptr<float>(), rows, cols, static_cast<float>(eps),
                       static_cast<float>(p), unpack_rng(rng), 0, dtype_code(x), cur_stream());
  return {y, z, mean, rstd};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> dropout_add_ln_bwd(
    const Tensor& gy, const optional<Tensor>& gz, const Tensor& z, const Tensor& gamma,
    const Tensor& mean, const Tensor& rstd, double p, const optional<Tensor>& rng,
    bool want_dbias) {
  check_cuda_contig(gy, "gy");
  check_cuda_contig(z, "z");
  c10::cuda::CUDAGuard guard(z.device());
  const int cols = static_cast<int>(z.size(-1));
  const int rows = static_cast<int>(z.numel() / cols);
  Tensor dx = at::empty_like(z);
  Tensor dres = p > 0.0 ? at::empty_like(z) : dx;
  Tensor dgamma = at::empty_like(gamma);
  Tensor dbeta = at::empty_like(gamma);
  Tensor dbias = at::empty({0}, z.options());
  if (want_dbias) dbias = at::empty_like(gamma);
  Tensor partial = at::empty({slapo::ln_bwd_grid(rows, cols), 3, cols},
                             z.options().dtype(at::kFloat));
  slapo::launch_ln_bwd(gy.data_ptr(), opt_ptr(gz), z.data_ptr(), gamma.data_ptr(),
                       mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(),
                       p > 0.0 ? dres.data_ptr() : nullptr, dgamma.data_ptr(), dbeta.data_ptr(),
                       want_dbias ? dbias.data_ptr() : nullptr, partial.data_ptr<float>(), rows,
                       cols, static_cast<float>(p), unpack_rng(rng), 0, dtype_code(z),
                       cur_stream());
  return {dx, dres, dgamma, dbeta, dbias};
}

// ------------------------------------------------------------------------ //
void fused_adamw(Tensor param, const Tensor& grad, Tensor master, Tensor exp_avg,
                 Tensor exp_avg_sq, const Tensor& decay_mask, const Tensor& grad_scale, double lr,
                 double beta1, double beta2, double eps, double weight_decay, double bc1,
                 double bc2, const optional<Tensor>& hyper) {
  check_cuda_contig(param, "param");
  check_cuda_contig(grad, "grad");
  check_cuda_contig(master, "master");
  c10::cuda::CUDAGuard guard(param.device());
  const int64_t n = param.numel();
  TORCH_CHECK(n % 8 == 0, "flat parameter length must be a multiple of 8");
  TORCH_CHECK(grad.numel() == n && master.numel() == n && exp_avg.numel() == n &&
              exp_avg_sq.numel() == n && decay_mask.numel() == n, "size mismatch");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(decay_mask.data_ptr()) % 8 == 0, "decay_mask alignment");
  slapo::launch_fused_adamw(param.data_ptr(), grad.data_ptr(), master.data_ptr<float>(),
                            exp_avg.data_ptr<float>(), exp_avg_sq.data_ptr<float>(),
                            decay_mask.data_ptr<uint8_t>(), grad_scale.data_ptr<float>(), n,
                            static_cast<float>(lr), static_cast<float>(beta1),
                            static_cast<float>(beta2), static_cast<float>(eps),
                            static_cast<float>(weight_decay), static_cast<float>(bc1),
                            static_cast<float>(bc2), dtype_code(param), cur_stream(),
                            hyper.has_value() && hyper->defined() ? hyper->data_ptr<float>()
                                                                  : nullptr);
}

}  // namespace

void register_gemm_ops(torch::Library& m);
void register_attn_ops(torch::Library& m);
void register_comm_ops(torch::Library& m);
void register_loss_ops(torch::Library& m);

TORCH_LIBRARY(slapo_b200, m) {
  m.def("philox_reserve(int increment) -> Tensor", &philox_reserve);
  m.def("launch_count() -> int", []() -> int64_t { return slapo::launch_count(); });
  m.def("bias_act_fwd(Tensor x, Tensor? bias, int act) -> Tensor", &bias_act_fwd);
  m.def("bias_act_bwd(Tensor dy, Tensor x, Tensor? bias, int act) -> (Tensor, Tensor)",
        &bias_act_bwd);
  m.def("act_bwd_colsum(Tensor dy, Tensor z, int act) -> (Tensor, Tensor)", &act_bwd_colsum);
  m.def("colsum(Tensor x) -> Tensor", &colsum);
  m.def("bias_dropout_add_fwd(Tensor x, Tensor? bias, Tensor? residual, float p, Tensor rng) -> Tensor",
        &bias_dropout_add_fwd);
  m.def("bias_dropout_add_bwd(Tensor dy, float p, Tensor rng, bool want_dbias) -> (Tensor, Tensor)",
        &bias_dropout_add_bwd);
  m.def("layer_norm_fwd(Tensor x, Tensor gamma, Tensor? beta, float eps, bool rms) -> (Tensor, Tensor, Tensor)",
        &layer_norm_fwd);
  m.def("layer_norm_bwd(Tensor gy, Tensor x, Tensor gamma, Tensor mean, Tensor rstd, bool rms) -> (Tensor, Tensor, Tensor)",
        &layer_norm_bwd);
  m.def("dropout_add_ln_fwd(Tensor x, Tensor? bias, Tensor residual, Tensor gamma, Tensor? beta, float p, float eps, Tensor? rng) -> (Tensor, Tensor, Tensor, Tensor)",
        &dropout_add_ln_fwd);
  m.def("dropout_add_ln_bwd(Tensor gy, Tensor? gz, Tensor z, Tensor gamma, Tensor mean, Tensor rstd, float p, Tensor? rng, bool want_dbias) -> (Tensor, Tensor, Tensor, Tensor, Tensor)",
        &dropout_add_ln_bwd);
  m.def("fused_adamw(Tensor(a!) param, Tensor grad, Tensor(b!) master, Tensor(c!) exp_avg, Tensor(d!) exp_avg_sq, Tensor decay_mask, Tensor grad_scale, float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2, Tensor? hyper=None) -> ()",
        &fused_adamw);
  register_gemm_ops(m);
  register_attn_ops(m);
  register_comm_ops(m);
  register_loss_ops(m);
}
