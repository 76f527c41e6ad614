// Host-side launchers of the sm_100a kernels.  Plain CUDA types only: the
// torch bindings (bindings.cpp) and stand-alone C callers share this header.
// dtype codes: 0 = bf16, 1 = fp16, 2 = fp32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace slapo {

struct PhiloxArgs;

// number of kernels launched by this library since load (host-side counter)
void count_launch(int n = 1);
int64_t launch_count();

int colsum_chunks(int rows, int cols);
int ln_bwd_grid(int rows, int cols);

void launch_bias_act_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols,
                         int act, int dtype, cudaStream_t stream);
void launch_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, void* dbias,
                         float* partial, int rows, int cols, int act, int dtype,
                         cudaStream_t stream);
// out[c] = sum over rows of x[r, c] (cols % 8 == 0); partial: colsum_chunks(rows, cols) * cols floats
void launch_colsum(const void* x, void* out, float* partial, int rows, int cols,
                   int64_t row_stride, int dtype, cudaStream_t stream);
void launch_colsum_finalize(const float* partial, void* out, int chunks, int cols, int dtype,
                            cudaStream_t stream);
void launch_fused_adamw(void* param, const void* grad, float* master, float* exp_avg,
                        float* exp_avg_sq, const uint8_t* decay_mask, const float* grad_scale,
                        int64_t n, float lr, float beta1, float beta2, float eps,
                        float weight_decay, float bc1, float bc2, int dtype, cudaStream_t stream,
                        const float* hyper = nullptr);

// C[M,N] = act(A B^T + bias); a_mn / b_mn select M/N-major operands (see gemm.cu).
// Returns 0 on success, >0 when the launch was refused on the host.
int launch_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                int lda, int ldb, int ldc, bool a_mn, bool b_mn, bool bf16, int act, int* status,
                cudaStream_t stream);

// The same product on CTA pairs (gemm2.cu): 256 x 256 tiles shared by two SMs, optional second
// output `C2` (the value before the activation), optional split-K through `workspace`
// (gemm2_splits() * M * N floats of scratch).  Returns 5 when
// the problem is smaller than one pair tile (use launch_gemm).
int gemm2_splits(int M, int N, int K, int bn);
int launch_gemm2(const void* A, const void* B, void* C, void* C2, const void* bias, int M, int N,
                 int K, int lda, int ldb, int ldc, bool a_mn, bool b_mn, bool bf16, int act,
                 float* workspace, int* status, cudaStream_t stream);

// Cross entropy in two steps (per-row statistics, then gradient); see loss.cu.
void launch_ce_stats(const void* logits, const int64_t* labels, float* stats, int rows, int cols,
                     int64_t row_stride, int vocab_start, int64_t ignore_index, int dtype,
                     cudaStream_t stream);
void launch_ce_grad(const void* logits, const int64_t* labels, const float* lse,
                    const float* coef, void* grad, int rows, int cols, int64_t row_stride,
                    int vocab_start, int64_t ignore_index, int dtype, cudaStream_t stream);
// out2[0] += sum x^2 where mask == 0 (or no mask), out2[1] += sum x^2 where mask == 1
// (elements with any other mask value are left out)
void launch_sq_norm(const void* x, const uint8_t* mask, float* out2, int64_t n, int dtype,
                    cudaStream_t stream);

// Fused GEMM + collective over peer memory (comm_gemm.cu).
//   gather: 0 none, 1 rows of A, 2 contraction dim of A, 3 contraction dim of B,
//           4 rows of A staged once through the local buffer stage_dst (chunk_flags: 2 * 8192
//             ints, zero-initialised, kept across calls - the epoch at which each 128-row
//             block was staged, then the slice counters of the same blocks)
//   mode:   0 local output, 1 reduce-scatter, 2 all-reduce
//   recv_mc / out_mc: NVLS addresses of the partial-product buffers (header first) and of the
//           all-reduce outputs, or null: the reduction then loads from every peer
int launch_comm_gemm(void* const* a_ptrs, void* const* b_ptrs, int M, int N, int K, int lda,
                     int ldb, bool a_mn, bool b_mn, bool bf16, int gather, int seg_len, int mode,
                     int world, int rank, int epoch, void* out, int ldo, const void* bias, int act,
                     int* flags, int* const* peer_flags, void* const* peer_recv,
                     void* const* peer_out, int* status, double wait_seconds, void* stage_dst,
                     int* chunk_flags, void* recv_mc, void* out_mc, void* const* stage_peers,
                     void* stage_mc, cudaStream_t stream);

// All-gather by peer stores (multicast through the NVSwitch when dst_mc is given): this rank's
// segment goes to offset rank * seg_bytes of every rank's buffer; the kernel ends when every
// rank's segment has landed in this rank's buffer.
int launch_peer_push_gather(const void* src, void* const* dst_ptrs, void* dst_mc, int64_t seg_bytes,
                            int world, int rank, int epoch, int* flags, int* const* peer_flags,
                            int* status, double wait_seconds, cudaStream_t stream);

// Phase trace of the last fused GEMM + collective kernel (recorded when the environment has
// SLAPO_B200_COMM_TRACE=1): [256 CTAs][8 slots] nanosecond time stamps, see comm_gemm.cu.
int read_comm_trace(unsigned long long* host, int n_words);

// dst = concatenation of every rank's segment, pulled over NVLink (comm_gemm.cu)
int launch_peer_gather(void* const* src_ptrs, void* dst, int64_t seg_bytes, int world, int rank,
                       int epoch, int* flags, int* const* peer_flags, int* status,
                       double wait_seconds, cudaStream_t stream);

// Data-parallel gradient reduce-scatter (pull) and AdamW + parameter all-gather (push) over
// peer memory (dp_comm.cu).  lo / n are element offsets / counts (multiples of 8) of this
// rank's slice inside the flat buffers; 16-bit dtypes only.
int launch_dp_grad_rs(void* const* grad_ptrs, int* const* flag_ptrs, int world, int rank,
                      int bucket, int epoch, int64_t lo, int64_t n, void* out,
                      const uint8_t* dup_mask, float* norm_acc, int* status, double wait_seconds,
                      int dtype, int phase, cudaStream_t stream);
int launch_dp_adamw_ag(void* const* param_ptrs, int* const* flag_ptrs, int world, int rank,
                       int n_buckets, int epoch, int last, int64_t lo, int64_t n, const void* grad,
                       float* master, float* exp_avg, float* exp_avg_sq, const uint8_t* decay_mask,
                       const float* grad_scale, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float bc1, float bc2, unsigned int* cta_counter,
                       int* status, double wait_seconds, int dtype, cudaStream_t stream);

// All-to-all of strided activation blocks by peer stores; strides and offsets in BYTES
// (multiples of 16).  Block j of src goes to dst_ptrs[j] + dst_block_offset.
int launch_peer_all_to_all(const void* src, void* const* dst_ptrs, int* const* flag_ptrs,
                           int world, int rank, int epoch, int outer, int rows, int row_bytes,
                           int64_t src_block_stride, int64_t src_outer_stride,
                           int64_t src_row_stride, int64_t dst_block_offset,
                           int64_t dst_outer_stride, int64_t dst_row_stride,
                           unsigned int* cta_counter, int* status, double wait_seconds,
                           cudaStream_t stream);

// Vocabulary-parallel embedding forward by peer stores (16-bit weights, hidden % 8 == 0).
// scatter: 0 = every rank receives every token's row; 1 = rank r keeps the r-th contiguous
// chunk of the tokens; 2 = rank r keeps the r-th chunk of every sequence of `seq` tokens
// (the sequence-parallel forms: out_ptrs then address [tokens / world, hidden] buffers).
int launch_vocab_embed_fwd(const int64_t* ids, const void* weight, void* const* out_ptrs,
                           int* const* flag_ptrs, int world, int rank, int epoch, int64_t tokens,
                           int hidden, int64_t vocab_lo, int64_t vocab_local, int scatter,
                           int64_t seq, unsigned int* cta_counter, int* status,
                           double wait_seconds, cudaStream_t stream);

}  // namespace slapo

#include "common_host.h"
