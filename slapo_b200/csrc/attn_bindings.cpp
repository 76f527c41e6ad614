// torch bindings of the tcgen05 flash-attention kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kernels.h"

int* slapo_status_ptr(int device);

namespace {

using at::Tensor;
using c10::optional;

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

void check_bshd(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 4, name, " must be a CUDA tensor [B, S, H, D]");
  TORCH_CHECK(t.stride(3) == 1, name, ": D must be contiguous");
  TORCH_CHECK(t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0,
              name, ": strides must be multiples of 8 elements");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

const float* opt_f32(const optional<Tensor>& t, const char* name) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous(), name,
              " must be a contiguous fp32 CUDA tensor");
  return t->data_ptr<float>();
}

std::tuple<Tensor, Tensor> flash_attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v,
                                          const optional<Tensor>& kbias,
                                          const optional<Tensor>& rel, bool causal, double scale,
                                          double p_drop, const optional<Tensor>& rng) {
  check_bshd(q, "q"); check_bshd(k, "k"); check_bshd(v, "v");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf, "bf16/fp16 only");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type());
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), Sq = q.size(1), H = q.size(2), D = q.size(3), Sk = k.size(1);
  TORCH_CHECK(k.size(0) == B && k.size(2) == H && k.size(3) == D && v.sizes() == k.sizes());
  if (kbias.has_value() && kbias->defined()) TORCH_CHECK(kbias->numel() == (int64_t)B * Sk);
  if (rel.has_value() && rel->defined()) TORCH_CHECK(rel->numel() == (int64_t)H * (Sq + Sk - 1));
  Tensor o = at::empty({B, Sq, H, D}, q.options());
  Tensor lse = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  const int64_t qs[3] = {q.stride(0), q.stride(1), q.stride(2)};
  const int64_t ks[3] = {k.stride(0), k.stride(1), k.stride(2)};
  const int64_t vs[3] = {v.stride(0), v.stride(1), v.stride(2)};
  int rc = slapo::launch_flash_fwd(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
      opt_f32(kbias, "key bias"), opt_f32(rel, "relative bias"), B, H, Sq, Sk, D, qs, ks, vs,
      static_cast<float>(scale), causal ? 1 : 0, static_cast<float>(p_drop), unpack_rng(rng),
      q.scalar_type() == at::kBFloat16, slapo_status_ptr(q.get_device()),
      at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "flash_attn_fwd: launch refused (code ", rc, ")");
  return {o, lse};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> flash_attn_bwd(
    const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
    const Tensor& lse, const optional<Tensor>& kbias, const optional<Tensor>& rel, bool causal,
    double scale, double p_drop, const optional<Tensor>& rng, bool packed_qkv) {
  check_bshd(q, "q"); check_bshd(k, "k"); check_bshd(v, "v");
  TORCH_CHECK(dout.is_contiguous() && o.is_contiguous(), "dout and out must be contiguous");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), Sq = q.size(1), H = q.size(2), D = q.size(3), Sk = k.size(1);
  // dQ: one fp32 partial per 128-key tile, written with plain stores and summed by the
  // conversion kernel (no zero fill, no atomics); beyond 16 key tiles, or 4 GB of partials,
  // a single zero-filled accumulator that the key tiles reduce into
  const int64_t n_kt = (Sk + 127) / 128;
  const int64_t dq_elems = static_cast<int64_t>(B) * Sq * H * D;
  const bool sliced = n_kt <= 16 && n_kt * dq_elems * 4 <= (int64_t(4) << 30);
  const int n_slices = sliced ? static_cast<int>(n_kt) : 1;
  Tensor dq_accum = sliced ? at::empty({n_kt, B, Sq, H, D}, q.options().dtype(at::kFloat))
                           : at::zeros({B, Sq, H, D}, q.options().dtype(at::kFloat));
  // packed_qkv: q, k, v are the slices [..., 0/1/2, :] of one [B, S, H, 3, D]
  // projection output; the gradients are written into one tensor of that
  // layout so that autograd needs no concatenation
  Tensor dk, dv, dqkv;
  int64_t dkv_stride = D;
  if (packed_qkv) {
    TORCH_CHECK(Sq == Sk, "packed QKV needs equal query and key lengths");
    dqkv = at::empty({B, Sq, H, 3, D}, q.options());
    dk = dqkv.select(3, 1);
    dv = dqkv.select(3, 2);
    dkv_stride = 3 * D;
  } else {
    dk = at::empty({B, Sk, H, D}, q.options());
    dv = at::empty({B, Sk, H, D}, q.options());
  }
  Tensor delta = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  Tensor drel;
  const bool has_rel = rel.has_value() && rel->defined();
  if (has_rel) drel = at::zeros_like(*rel);
  else drel = at::empty({0}, q.options().dtype(at::kFloat));
  const int64_t qs[3] = {q.stride(0), q.stride(1), q.stride(2)};
  const int64_t ks[3] = {k.stride(0), k.stride(1), k.stride(2)};
  const int64_t vs[3] = {v.stride(0), v.stride(1), v.stride(2)};
  int rc = slapo::launch_flash_bwd(
      q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
      lse.data_ptr<float>(), delta.data_ptr<float>(), dq_accum.data_ptr<float>(),
      sliced ? dq_elems : 0, dk.data_ptr(), dv.data_ptr(), dkv_stride, opt_f32(kbias, "key bias"), opt_f32(rel, "relative bias"),
      has_rel ? drel.data_ptr<float>() : nullptr, B, H, Sq, Sk, D, qs, ks, vs,
      static_cast<float>(scale), causal ? 1 : 0, static_cast<float>(p_drop), unpack_rng(rng),
      q.scalar_type() == at::kBFloat16, slapo_status_ptr(q.get_device()),
      at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "flash_attn_bwd: launch refused (code ", rc, ")");
  const bool bf16 = q.scalar_type() == at::kBFloat16;
  const int64_t rows = static_cast<int64_t>(B) * Sq * H;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  if (packed_qkv) {
    // dq is slice 0 of the packed gradient: rows of D values, 3 D apart
    slapo::launch_flash_dq_convert(dq_accum.data_ptr<float>(), dqkv.data_ptr(), rows, D, 3 * D,
                                   bf16, n_slices, dq_elems, Sq, Sk, H, causal ? 1 : 0, stream);
    return {dqkv, dk, dv, drel};
  }
  Tensor dq = at::empty({B, Sq, H, D}, q.options());
  slapo::launch_flash_dq_convert(dq_accum.data_ptr<float>(), dq.data_ptr(), rows, D, D, bf16,
                                 n_slices, dq_elems, Sq, Sk, H, causal ? 1 : 0, stream);
  return {dq, dk, dv, drel};
}

Tensor flash_attn_dropout_mask(int64_t B, int64_t H, int64_t Sq, int64_t Sk, double p_drop,
                               const Tensor& rng) {
  Tensor mask = at::empty({B, H, Sq, Sk}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA));
  slapo::launch_flash_dropout_mask(mask.data_ptr<uint8_t>(), B, H, Sq, Sk,
                                   static_cast<float>(p_drop), unpack_rng(rng),
                                   at::cuda::getCurrentCUDAStream().stream());
  return mask;
}

}  // namespace

void register_attn_ops(torch::Library& m) {
  m.def("flash_attn_fwd(Tensor q, Tensor k, Tensor v, Tensor? kbias, Tensor? rel, bool causal, float scale, float p_drop, Tensor? rng) -> (Tensor, Tensor)",
        &flash_attn_fwd);
  m.def("flash_attn_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, Tensor? kbias, Tensor? rel, bool causal, float scale, float p_drop, Tensor? rng, bool packed_qkv) -> (Tensor, Tensor, Tensor, Tensor)",
        &flash_attn_bwd);
  m.def("flash_attn_dropout_mask(int B, int H, int Sq, int Sk, float p_drop, Tensor rng) -> Tensor",
        &flash_attn_dropout_mask);
}
