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
               int64_t chunk_flags_ptr) {
  TORCH_CHECK(!a_ptrs.empty() && !b_ptrs.empty(), "comm_gemm: operand pointers missing");
  auto a = to_ptrs<void*>(a_ptrs);
  auto b = to_ptrs<void*>(b_ptrs);
  auto pf = to_ptrs<int*>(peer_flags);
  auto pr = to_ptrs<void*>(peer_recv);
  auto po = to_ptrs<void*>(peer_out);
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
      reinterpret_cast<int*>(chunk_flags_ptr), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "comm_gemm: launch refused (code ", rc,
              "): check divisibility by the group size / 128-row blocks and 16-byte alignment");
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

}  // namespace

void register_comm_ops(torch::Library& m) {
  m.def("comm_gemm(int[] a_ptrs, int[] b_ptrs, int M, int N, int K, int lda, int ldb, bool a_mn, "
        "bool b_mn, bool bf16, int gather, int seg_len, int mode, int world, int rank, int epoch, "
        "int out_ptr, int ldo, int bias_ptr, int act, int flags_ptr, int[] peer_flags, "
        "int[] peer_recv, int[] peer_out, float wait_seconds, int stage_ptr, "
        "int chunk_flags_ptr) -> ()", &comm_gemm);
  m.def("peer_gather(int[] src_ptrs, int dst_ptr, int seg_bytes, int world, int rank, int epoch, "
        "int flags_ptr, int[] peer_flags, float wait_seconds) -> ()", &peer_gather);
}
