// torch bindings of the fused compute+collective kernels.  Buffers that live
// in other ranks' memory have no tensor on this rank, so operands are passed
// as raw device addresses; the Python side keeps the owning tensors alive.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kernels.h"

int* slapo_status_ptr(int device);

namespace {

template <typename T>
std::vector<T> to_ptrs(const std::vector<int64_t>& v) {
  std::vector<T> out(8, nullptr);
  for (size_t i = 0; i < v.size() && i < 8; ++i) out[i] = reinterpret_cast<T>(v[i]);
  return out;
}

void comm_gemm(std::vector<int64_t> a_ptrs, std::vector<int64_t> b_ptrs, int64_t M, int64_t N,
               int64_t K, int64_t lda, int64_t ldb, bool a_mn, bool b_mn, bool bf16,
               int64_t gather, int64_t seg_len, int64_t mode, int64_t world, int64_t rank,
               int64_t epoch, int64_t out_ptr, int64_t ldo, int64_t bias_ptr, int64_t act,
               int64_t flags_ptr, std::vector<int64_t> peer_flags, std::vector<int64_t> peer_recv,
               std::vector<int64_t> peer_out, double wait_seconds, int64_t stage_ptr,
               int64_t chunk_flags_ptr, int64_t recv_mc, int64_t out_mc,
               std::vector<int64_t> stage_peers, int64_t stage_mc) {
  TORCH_CHECK(!a_ptrs.empty() && !b_ptrs.empty(), "comm_gemm: operand pointers missing");
  auto a = to_ptrs<void*>(a_ptrs);
  auto b = to_ptrs<void*>(b_ptrs);
  auto pf = to_ptrs<int*>(peer_flags);
  auto pr = to_ptrs<void*>(peer_recv);
  auto po = to_ptrs<void*>(peer_out);
  auto sp = to_ptrs<void*>(stage_peers);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_comm_gemm(
      a.data(), b.data(), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
      static_cast<int>(lda), static_cast<int>(ldb), a_mn, b_mn, bf16, static_cast<int>(gather),
      static_cast<int>(seg_len), static_cast<int>(mode), static_cast<int>(world),
      static_cast<int>(rank), static_cast<int>(epoch), reinterpret_cast<void*>(out_ptr),
      static_cast<int>(ldo), reinterpret_cast<const void*>(bias_ptr), static_cast<int>(act),
      reinterpret_cast<int*>(flags_ptr), peer_flags.empty() ? nullptr : pf.data(),
      peer_recv.empty() ? nullptr : pr.data(), peer_out.empty() ? nullptr : po.data(),
      slapo_status_ptr(dev), wait_seconds, reinterpret_cast<void*>(stage_ptr),
      reinterpret_cast<int*>(chunk_flags_ptr), reinterpret_cast<void*>(recv_mc),
      reinterpret_cast<void*>(out_mc), stage_peers.empty() ? nullptr : sp.data(),
      reinterpret_cast<void*>(stage_mc), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "comm_gemm: launch refused (code ", rc,
              "): check divisibility by the group size / 128-row blocks and 16-byte alignment");
}

at::Tensor comm_trace() {
  auto out = at::zeros({256, 8}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
  at::cuda::getCurrentCUDAStream().synchronize();
  TORCH_CHECK(slapo::read_comm_trace(reinterpret_cast<unsigned long long*>(out.data_ptr<int64_t>()),
                                     256 * 8) == 0, "reading the phase trace failed");
  return out;
}

void peer_gather(std::vector<int64_t> src_ptrs, int64_t dst_ptr, int64_t seg_bytes, int64_t world,
                 int64_t rank, int64_t epoch, int64_t flags_ptr, std::vector<int64_t> peer_flags,
                 double wait_seconds) {
  auto src = to_ptrs<void*>(src_ptrs);
  auto pf = to_ptrs<int*>(peer_flags);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_peer_gather(
      src.data(), reinterpret_cast<void*>(dst_ptr), seg_bytes, static_cast<int>(world),
      static_cast<int>(rank), static_cast<int>(epoch), reinterpret_cast<int*>(flags_ptr),
      peer_flags.empty() ? nullptr : pf.data(), slapo_status_ptr(dev), wait_seconds,
      at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "peer_gather: launch refused (code ", rc, ")");
}

void peer_push_gather(int64_t src_ptr, std::vector<int64_t> dst_ptrs, int64_t dst_mc,
                      int64_t seg_bytes, int64_t world, int64_t rank, int64_t epoch,
                      int64_t flags_ptr, std::vector<int64_t> peer_flags, double wait_seconds) {
  auto dst = to_ptrs<void*>(dst_ptrs);
  auto pf = to_ptrs<int*>(peer_flags);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_peer_push_gather(
      reinterpret_cast<const void*>(src_ptr), dst.data(), reinterpret_cast<void*>(dst_mc), seg_bytes,
      static_cast<int>(world), static_cast<int>(rank), static_cast<int>(epoch),
      reinterpret_cast<int*>(flags_ptr), peer_flags.empty() ? nullptr : pf.data(),
      slapo_status_ptr(dev), wait_seconds, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "peer_push_gather: launch refused (code ", rc, ")");
}

int dtype16(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf,
              "fused data-parallel kernels need bf16 or fp16 parameters");
  return t.scalar_type() == at::kBFloat16 ? 0 : 1;
}

// out <- mean over ranks of grads[lo : lo + out.numel()] pulled from every rank's flat gradient
void dp_grad_rs(std::vector<int64_t> grad_ptrs, std::vector<int64_t> flag_ptrs, int64_t world,
                int64_t rank, int64_t bucket, int64_t epoch, int64_t lo, at::Tensor out,
                const c10::optional<at::Tensor>& dup_mask,
                const c10::optional<at::Tensor>& norm_acc, double wait_seconds, int64_t phase) {
  c10::cuda::CUDAGuard guard(out.device());
  auto g = to_ptrs<void*>(grad_ptrs);
  auto f = to_ptrs<int*>(flag_ptrs);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_dp_grad_rs(
      g.data(), f.data(), static_cast<int>(world), static_cast<int>(rank),
      static_cast<int>(bucket), static_cast<int>(epoch), lo, out.numel(), out.data_ptr(),
      dup_mask.has_value() && dup_mask->defined() ? dup_mask->data_ptr<uint8_t>() : nullptr,
      norm_acc.has_value() && norm_acc->defined() ? norm_acc->data_ptr<float>() : nullptr,
      slapo_status_ptr(dev), wait_seconds, dtype16(out), static_cast<int>(phase),
      at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "dp_grad_rs: launch refused (code ", rc, ")");
}

// AdamW on this rank's slice, new parameters written to every rank's flat parameter buffer
void dp_adamw_ag(std::vector<int64_t> param_ptrs, std::vector<int64_t> flag_ptrs, int64_t world,
                 int64_t rank, int64_t n_buckets, int64_t epoch, bool last, int64_t lo,
                 at::Tensor grad, at::Tensor master, at::Tensor exp_avg, at::Tensor exp_avg_sq,
                 at::Tensor decay_mask, at::Tensor grad_scale, double lr, double beta1,
                 double beta2, double eps, double weight_decay, double bc1, double bc2,
                 at::Tensor cta_counter, double wait_seconds) {
  c10::cuda::CUDAGuard guard(grad.device());
  auto p = to_ptrs<void*>(param_ptrs);
  auto f = to_ptrs<int*>(flag_ptrs);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_dp_adamw_ag(
      p.data(), f.data(), static_cast<int>(world), static_cast<int>(rank),
      static_cast<int>(n_buckets), static_cast<int>(epoch), last ? 1 : 0, lo, grad.numel(),
      grad.data_ptr(), master.data_ptr<float>(), exp_avg.data_ptr<float>(),
      exp_avg_sq.data_ptr<float>(), decay_mask.data_ptr<uint8_t>(), grad_scale.data_ptr<float>(),
      static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
      static_cast<float>(eps), static_cast<float>(weight_decay), static_cast<float>(bc1),
      static_cast<float>(bc2), reinterpret_cast<unsigned int*>(cta_counter.data_ptr<int>()),
      slapo_status_ptr(dev), wait_seconds, dtype16(grad), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "dp_adamw_ag: launch refused (code ", rc, ")");
}

void peer_all_to_all(at::Tensor src, std::vector<int64_t> dst_ptrs, std::vector<int64_t> flag_ptrs,
                     int64_t world, int64_t rank, int64_t epoch, int64_t outer, int64_t rows,
                     int64_t row_bytes, int64_t src_block_stride, int64_t src_outer_stride,
                     int64_t src_row_stride, int64_t dst_block_offset, int64_t dst_outer_stride,
                     int64_t dst_row_stride, at::Tensor cta_counter, double wait_seconds) {
  c10::cuda::CUDAGuard guard(src.device());
  auto d = to_ptrs<void*>(dst_ptrs);
  auto f = to_ptrs<int*>(flag_ptrs);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_peer_all_to_all(
      src.data_ptr(), d.data(), f.data(), static_cast<int>(world), static_cast<int>(rank),
      static_cast<int>(epoch), static_cast<int>(outer), static_cast<int>(rows),
      static_cast<int>(row_bytes), src_block_stride, src_outer_stride, src_row_stride,
      dst_block_offset, dst_outer_stride, dst_row_stride,
      reinterpret_cast<unsigned int*>(cta_counter.data_ptr<int>()), slapo_status_ptr(dev),
      wait_seconds, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "peer_all_to_all: launch refused (code ", rc,
              "): rows and strides must be multiples of 16 bytes");
}

void vocab_embed_fwd(at::Tensor ids, at::Tensor weight, std::vector<int64_t> out_ptrs,
                     std::vector<int64_t> flag_ptrs, int64_t world, int64_t rank, int64_t epoch,
                     int64_t vocab_lo, at::Tensor cta_counter, double wait_seconds,
                     int64_t scatter, int64_t seq) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(),
              "vocab_embed_fwd: ids must be a contiguous CUDA int64 tensor");
  TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous() && weight.element_size() == 2,
              "vocab_embed_fwd: weight must be a contiguous 16-bit [vocab_local, hidden] tensor");
  c10::cuda::CUDAGuard guard(weight.device());
  auto o = to_ptrs<void*>(out_ptrs);
  auto f = to_ptrs<int*>(flag_ptrs);
  const int dev = at::cuda::current_device();
  int rc = slapo::launch_vocab_embed_fwd(
      ids.data_ptr<int64_t>(), weight.data_ptr(), o.data(), f.data(), static_cast<int>(world),
      static_cast<int>(rank), static_cast<int>(epoch), ids.numel(),
      static_cast<int>(weight.size(1)), vocab_lo, weight.size(0), static_cast<int>(scatter), seq,
      reinterpret_cast<unsigned int*>(cta_counter.data_ptr<int>()), slapo_status_ptr(dev),
      wait_seconds, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "vocab_embed_fwd: launch refused (code ", rc, ")");
}

}  // namespace

void register_comm_ops(torch::Library& m) {
  m.def("vocab_embed_fwd(Tensor ids, Tensor weight, int[] out_ptrs, int[] flag_ptrs, int world, "
        "int rank, int epoch, int vocab_lo, Tensor(a!) cta_counter, float wait_seconds, "
        "int scatter=0, int seq=0) -> ()",
        &vocab_embed_fwd);
  m.def("peer_all_to_all(Tensor src, int[] dst_ptrs, int[] flag_ptrs, int world, int rank, "
        "int epoch, int outer, int rows, int row_bytes, int src_block_stride, "
        "int src_outer_stride, int src_row_stride, int dst_block_offset, int dst_outer_stride, "
        "int dst_row_stride, Tensor(a!) cta_counter, float wait_seconds) -> ()", &peer_all_to_all);
  m.def("dp_grad_rs(int[] grad_ptrs, int[] flag_ptrs, int world, int rank, int bucket, int epoch, "
        "int lo, Tensor(a!) out, Tensor? dup_mask, Tensor(b!)? norm_acc, float wait_seconds, "
        "int phase) -> ()",
        &dp_grad_rs);
  m.def("dp_adamw_ag(int[] param_ptrs, int[] flag_ptrs, int world, int rank, int n_buckets, "
        "int epoch, bool last, int lo, Tensor grad, Tensor(a!) master, Tensor(b!) exp_avg, "
        "Tensor(c!) exp_avg_sq, Tensor decay_mask, Tensor grad_scale, float lr, float beta1, "
        "float beta2, float eps, float weight_decay, float bc1, float bc2, Tensor(d!) cta_counter, "
        "float wait_seconds) -> ()", &dp_adamw_ag);
  m.def("comm_gemm(int[] a_ptrs, int[] b_ptrs, int M, int N, int K, int lda, int ldb, bool a_mn, "
        "bool b_mn, bool bf16, int gather, int seg_len, int mode, int world, int rank, int epoch, "
        "int out_ptr, int ldo, int bias_ptr, int act, int flags_ptr, int[] peer_flags, "
        "int[] peer_recv, int[] peer_out, float wait_seconds, int stage_ptr, "
        "int chunk_flags_ptr, int recv_mc, int out_mc, int[] stage_peers, int stage_mc) -> ()",
        &comm_gemm);
  m.def("comm_trace() -> Tensor", &comm_trace);
  m.def("peer_push_gather(int src_ptr, int[] dst_ptrs, int dst_mc, int seg_bytes, int world, "
        "int rank, int epoch, int flags_ptr, int[] peer_flags, float wait_seconds) -> ()",
        &peer_push_gather);
  m.def("peer_gather(int[] src_ptrs, int dst_ptr, int seg_bytes, int world, int rank, int epoch, "
        "int flags_ptr, int[] peer_flags, float wait_seconds) -> ()", &peer_gather);
}
