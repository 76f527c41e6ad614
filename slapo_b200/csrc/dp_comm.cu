// Data-parallel collectives fused with the optimizer, over NVLink peer memory.
//
// Every rank keeps its flat gradient and flat parameter buffers in symmetric
// memory (same offset on every GPU).  One training step needs two kernels per
// gradient bucket instead of reduce-scatter + AdamW + all-gather launches:
//
//   dp_grad_rs_kernel   (launched on the communication stream as soon as the
//                        backward pass has finished a bucket)
//       publishes "my gradients of this bucket are final", waits - bounded -
//       for the same from every peer, then PULLS its own slice of the bucket
//       from every peer, averages in fp32, writes the reduced slice and
//       accumulates the squared gradient norm (split into tensor-parallel
//       sharded / replicated parts) for clipping;
//
//   dp_adamw_ag_kernel  (after the clip coefficient is known)
//       AdamW on the owned slice with fp32 master weights and moments and
//       PUSHES the new 16-bit parameters into every rank's parameter buffer
//       (the all-gather).  In the last bucket the CTA that finishes last
//       publishes "pushed" and waits for the peers' "pushed" flags, so when the
//       kernel completes every rank's slice has landed here and every peer has
//       finished reading this rank's gradients (they may be zeroed).
//
// Flags live in a symmetric int array: slot (bucket, rank) for "ready",
// slot (n_buckets, rank) for "pushed"; values are the step number, monotone.
// Every wait is bounded: on expiry the status word is set and the kernel ends.
#include "common.cuh"
#include "kernels.h"

namespace slapo {

constexpr int kDpMaxRanks = 8;

struct DpPeers {
  void* ptr[kDpMaxRanks];
};
struct DpFlagPeers {
  int* ptr[kDpMaxRanks];
};

__device__ __forceinline__ void dp_st_release(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int dp_ld_acquire(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ bool dp_wait(const int* addr, int epoch, long long budget) {
  if (dp_ld_acquire(addr) >= epoch) return true;
  const long long start = clock64();
  while (dp_ld_acquire(addr) < epoch) {
    if (clock64() - start > budget) return false;
    __nanosleep(128);
  }
  return true;
}

// 16-byte load that does not allocate in L1 (peer data is read exactly once)
template <typename T>
__device__ __forceinline__ void load8_stream(const T* p, float v[8]) {
  uint4 raw;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
               : "l"(p));
  if constexpr (sizeof(T) == 2) {
    Vec8<T>::load(reinterpret_cast<const T*>(&raw), v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dp_grad_rs_kernel(
    DpPeers grads, DpFlagPeers flags, int world, int rank, int bucket, int epoch, int64_t lo,
    int64_t n_vec, T* __restrict__ out, const uint8_t* __restrict__ dup_mask,
    float* __restrict__ norm_acc, int* __restrict__ status, long long wait_cycles, int phase) {
  // phase 0: handshake + pull in one launch; 1: handshake only (a single small CTA, so that a
  // wait for a slow peer does not occupy the SMs the backward pass is using); 2: pull only
  __shared__ int s_ok;
  __shared__ float s_red[2][8];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (phase != 2) {
    // 1. publish (one CTA) and wait for the peers (every CTA)
    if (blockIdx.x == 0 && threadIdx.x < world && threadIdx.x != rank) {
      __threadfence_system();
      dp_st_release(flags.ptr[threadIdx.x] + bucket * kDpMaxRanks + rank, epoch);
    }
    if (threadIdx.x < world && threadIdx.x != rank) {
      if (!dp_wait(flags.ptr[rank] + bucket * kDpMaxRanks + threadIdx.x, epoch, wait_cycles)) {
        s_ok = 0;
        atomicExch(status, 5);
      }
    }
    __syncthreads();
    if (!s_ok || phase == 1) return;
  }
  // 2. pull, average, write, norm
  const float inv_world = 1.f / static_cast<float>(world);
  float sq_shard = 0.f, sq_dup = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += stride) {
    const int64_t e = lo + i * kVec;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float v[kDpMaxRanks][8];
#pragma unroll
    for (int r = 0; r < kDpMaxRanks; ++r) {
      if (r < world) {
        // start with the peer after this rank so the ranks do not all read one GPU at once
        int src = rank + r;
        if (src >= world) src -= world;
        load8_stream(static_cast<const T*>(grads.ptr[src]) + e, v[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kDpMaxRanks; ++r) {
      if (r < world) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += v[r][k];
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= inv_world;
    Vec8<T>::store(out + i * kVec, acc);
    round_through<T>(acc);  // the norm of what the optimizer will read
    if (dup_mask != nullptr) {
      const uint2 dm = *reinterpret_cast<const uint2*>(dup_mask + i * kVec);
      const uint8_t* dmb = reinterpret_cast<const uint8_t*>(&dm);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (dmb[k] == 1) sq_dup += acc[k] * acc[k];
        else if (dmb[k] == 0) sq_shard += acc[k] * acc[k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) sq_shard += acc[k] * acc[k];
    }
  }
  if (norm_acc != nullptr) {
    sq_shard = warp_sum(sq_shard);
    sq_dup = warp_sum(sq_dup);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_red[0][warp] = sq_shard; s_red[1][warp] = sq_dup; }
    __syncthreads();
    if (threadIdx.x < 2) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += s_red[threadIdx.x][w];
      atomicAdd(norm_acc + threadIdx.x, t);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dp_adamw_ag_kernel(
    DpPeers params, DpFlagPeers flags, int world, int rank, int n_buckets, int epoch, int last,
    int64_t lo, int64_t n_vec, const T* __restrict__ grad, float* __restrict__ master,
    float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
    const uint8_t* __restrict__ decay_mask, const float* __restrict__ grad_scale, float lr,
    float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
    unsigned int* __restrict__ cta_counter, int* __restrict__ status, long long wait_cycles) {
  const float gs = grad_scale != nullptr ? *grad_scale : 1.f;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += stride) {
    const int64_t e = i * kVec;
    float g[8], w[8], m[8], v[8];
    Vec8<T>::load(grad + e, g);
    Vec8<float>::load(master + e, w);
    Vec8<float>::load(exp_avg + e, m);
    Vec8<float>::load(exp_avg_sq + e, v);
    const uint2 dm = *reinterpret_cast<const uint2*>(decay_mask + e);
    const uint8_t* dmb = reinterpret_cast<const uint8_t*>(&dm);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * gs;
      m[k] = beta1 * m[k] + (1.f - beta1) * gk;
      v[k] = beta2 * v[k] + (1.f - beta2) * gk * gk;
      const float denom = sqrtf(v[k]) * inv_sqrt_bc2 + eps;
      float upd = (m[k] * inv_bc1) / denom;
      if (dmb[k]) upd += weight_decay * w[k];
      w[k] -= lr * upd;
    }
    Vec8<float>::store(master + e, w);
    Vec8<float>::store(exp_avg + e, m);
    Vec8<float>::store(exp_avg_sq + e, v);
    // the all-gather: the new parameters go to every rank's buffer, this rank's first
#pragma unroll
    for (int r = 0; r < kDpMaxRanks; ++r) {
      if (r < world) {
        int dst = rank + r;
        if (dst >= world) dst -= world;
        Vec8<T>::store(static_cast<T*>(params.ptr[dst]) + lo + e, w);
      }
    }
  }
  if (!last) return;
  // 3. end of step: the CTA that finishes last tells the peers and waits for them
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(cta_counter, 1u);
    s_last = (done == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) *cta_counter = 0u;  // ready for the next step
  if (threadIdx.x < world && threadIdx.x != rank) {
    __threadfence_system();
    dp_st_release(flags.ptr[threadIdx.x] + n_buckets * kDpMaxRanks + rank, epoch);
    if (!dp_wait(flags.ptr[rank] + n_buckets * kDpMaxRanks + threadIdx.x, epoch, wait_cycles))
      atomicExch(status, 6);
  }
}

// ------------------------------------------------------------------------ //
// All-to-all of activation blocks by peer stores (the RS <-> SR reshard).
// Rank r's block for rank j is a strided 3-D box [outer, rows, row_vecs * 8]; it lands in
// rank j's receive buffer at the position that concatenation along the other axis asks for,
// so neither side needs a packing or an un-packing copy.  The CTA that finishes last
// publishes "sent" to every peer and waits (bounded) for theirs: when the kernel ends, this
// rank's receive buffer is complete.
struct A2AParams {
  const void* src;
  void* dst[kDpMaxRanks];       // every rank's receive buffer
  int* flags[kDpMaxRanks];      // every rank's flag pad (slots 0..7: sent by rank i)
  int world, rank, epoch;
  int outer, rows, row_vecs;    // box extent (row_vecs in 16-byte vectors)
  // element offsets (in 16-byte vectors) of block j inside src, and of this rank's block
  // inside a destination buffer
  int64_t src_block_stride, src_outer_stride, src_row_stride;
  int64_t dst_block_offset, dst_outer_stride, dst_row_stride;
  unsigned int* cta_counter;
  int* status;
  long long wait_cycles;
};

__global__ void __launch_bounds__(256) peer_all_to_all_kernel(A2AParams p) {
  const int64_t per_block = static_cast<int64_t>(p.outer) * p.rows * p.row_vecs;
  const int64_t total = per_block * p.world;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint4* src = static_cast<const uint4*>(p.src);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    int j = static_cast<int>(i / per_block);         // destination slot, rotated below
    int64_t rem = i - j * per_block;
    const int v = static_cast<int>(rem % p.row_vecs);
    rem /= p.row_vecs;
    const int r = static_cast<int>(rem % p.rows);
    const int o = static_cast<int>(rem / p.rows);
    j += p.rank;                                     // start with the own block, then rank + 1 ...
    if (j >= p.world) j -= p.world;
    const uint4 val = src[j * p.src_block_stride + o * p.src_outer_stride + r * p.src_row_stride + v];
    static_cast<uint4*>(p.dst[j])[p.dst_block_offset + o * p.dst_outer_stride +
                                  r * p.dst_row_stride + v] = val;
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(p.cta_counter, 1u);
    s_last = (done == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) *p.cta_counter = 0u;
  if (threadIdx.x < p.world && threadIdx.x != p.rank) {
    __threadfence_system();
    dp_st_release(p.flags[threadIdx.x] + p.rank, p.epoch);
    if (!dp_wait(p.flags[p.rank] + threadIdx.x, p.epoch, p.wait_cycles)) atomicExch(p.status, 7);
  }
}

// ------------------------------------------------------------------------ //
// ------------------------------------------------------------------------ //
// Vocabulary-parallel embedding forward without an all-reduce: exactly one rank owns the
// row of each token id, so that rank stores the row straight into EVERY rank's output
// (peer stores); ranks that do not own an id write nothing.  One warp per token.  The
// last CTA to finish exchanges "sent" flags with the peers (bounded wait): when the kernel
// ends this rank's output holds every row.
// Sequence-parallel form (`scatter` != 0): a rank keeps only ITS tokens, so the owner of a
// row stores it into the one rank that keeps the token - the reduce-scatter of the masked
// lookups, without the lookups of zeros and without the reduction.  scatter 1: tokens are
// split in `world` contiguous chunks (batch-major activations split along the batch);
// scatter 2: every sequence of `seq` tokens is split in `world` chunks.
struct VocabEmbedParams {
  const int64_t* ids;
  const void* weight;           // [vocab_local, hidden] 16-bit
  void* out[kDpMaxRanks];       // every rank's [tokens, hidden] output buffer
  int* flags[kDpMaxRanks];
  int world, rank, epoch;
  int64_t tokens;
  int hidden_vecs;              // hidden * 2 / 16
  int64_t vocab_lo, vocab_local;
  int scatter;                  // 0 every rank gets every row, 1 / 2 see above
  int64_t seq;                  // scatter 2: tokens per sequence
  unsigned int* cta_counter;
  int* status;
  long long wait_cycles;
};

__global__ void __launch_bounds__(256) vocab_embed_fwd_kernel(VocabEmbedParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp; t < p.tokens;
       t += warps) {
    const int64_t id = p.ids[t] - p.vocab_lo;
    if (id < 0 || id >= p.vocab_local) continue;   // another rank owns this row
    const uint4* src = static_cast<const uint4*>(p.weight) + id * p.hidden_vecs;
    if (p.scatter != 0) {
      int dst;
      int64_t row;
      if (p.scatter == 1) {
        const int64_t per = p.tokens / p.world;
        dst = static_cast<int>(t / per);
        row = t - dst * per;
      } else {
        const int64_t per = p.seq / p.world, s_pos = t % p.seq;
        dst = static_cast<int>(s_pos / per);
        row = (t / p.seq) * per + (s_pos - dst * per);
      }
      uint4* out = static_cast<uint4*>(p.out[dst]) + row * p.hidden_vecs;
      for (int v = lane; v < p.hidden_vecs; v += 32) out[v] = src[v];
      continue;
    }
    for (int v = lane; v < p.hidden_vecs; v += 32) {
      const uint4 val = src[v];
#pragma unroll
      for (int r = 0; r < kDpMaxRanks; ++r) {
        if (r < p.world) {
          int dst = p.rank + r;
          if (dst >= p.world) dst -= p.world;
          static_cast<uint4*>(p.out[dst])[t * p.hidden_vecs + v] = val;
        }
      }
    }
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(p.cta_counter, 1u);
    s_last = (done == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) *p.cta_counter = 0u;
  if (threadIdx.x < p.world && threadIdx.x != p.rank) {
    __threadfence_system();
    dp_st_release(p.flags[threadIdx.x] + p.rank, p.epoch);
    if (!dp_wait(p.flags[p.rank] + threadIdx.x, p.epoch, p.wait_cycles)) atomicExch(p.status, 8);
  }
}

// clock64() ticks at the SM clock; its maximum (1.965 GHz on B200) turns seconds into a
// cycle budget.  A constant on purpose: querying the clock-rate attribute costs about a
// millisecond per call, which is more than the kernels these budgets guard.
static long long dp_wait_cycles(double seconds) {
  return static_cast<long long>(seconds * 1.965e9);
}

static int dp_grid(int64_t n_vec) {
  int64_t blocks = (n_vec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks > 0 ? blocks : 1);
}

int launch_dp_grad_rs(void* const* grad_ptrs, int* const* flag_ptrs, int world, int rank,
                      int bucket, int epoch, int64_t lo, int64_t n, void* out,
                      const uint8_t* dup_mask, float* norm_acc, int* status, double wait_seconds,
                      int dtype, int phase, cudaStream_t stream) {
  if (world < 1 || world > kDpMaxRanks || n % kVec != 0 || lo % kVec != 0) return 1;
  if (dtype != 0 && dtype != 1) return 2;  // 16-bit gradients only
  DpPeers g;
  DpFlagPeers f;
  for (int r = 0; r < kDpMaxRanks; ++r) {
    g.ptr[r] = r < world ? grad_ptrs[r] : nullptr;
    f.ptr[r] = r < world ? flag_ptrs[r] : nullptr;
  }
  const int64_t n_vec = n / kVec;
  const long long cycles = dp_wait_cycles(wait_seconds);
  const int grid = phase == 1 ? 1 : dp_grid(n_vec);
  const int block = phase == 1 ? 32 : 256;
  count_launch();
  if (dtype == 0)
    dp_grad_rs_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        g, f, world, rank, bucket, epoch, lo, n_vec, static_cast<__nv_bfloat16*>(out), dup_mask,
        norm_acc, status, cycles, phase);
  else
    dp_grad_rs_kernel<__half><<<grid, block, 0, stream>>>(
        g, f, world, rank, bucket, epoch, lo, n_vec, static_cast<__half*>(out), dup_mask, norm_acc,
        status, cycles, phase);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int launch_dp_adamw_ag(void* const* param_ptrs, int* const* flag_ptrs, int world, int rank,
                       int n_buckets, int epoch, int last, int64_t lo, int64_t n, const void* grad,
                       float* master, float* exp_avg, float* exp_avg_sq, const uint8_t* decay_mask,
                       const float* grad_scale, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float bc1, float bc2, unsigned int* cta_counter,
                       int* status, double wait_seconds, int dtype, cudaStream_t stream) {
  if (world < 1 || world > kDpMaxRanks || n % kVec != 0 || lo % kVec != 0) return 1;
  if (dtype != 0 && dtype != 1) return 2;
  DpPeers p;
  DpFlagPeers f;
  for (int r = 0; r < kDpMaxRanks; ++r) {
    p.ptr[r] = r < world ? param_ptrs[r] : nullptr;
    f.ptr[r] = r < world ? flag_ptrs[r] : nullptr;
  }
  const int64_t n_vec = n / kVec;
  const long long cycles = dp_wait_cycles(wait_seconds);
  count_launch();
  if (dtype == 0)
    dp_adamw_ag_kernel<__nv_bfloat16><<<dp_grid(n_vec), 256, 0, stream>>>(
        p, f, world, rank, n_buckets, epoch, last, lo, n_vec, static_cast<const __nv_bfloat16*>(grad),
        master, exp_avg, exp_avg_sq, decay_mask, grad_scale, lr, beta1, beta2, eps, weight_decay,
        bc1, bc2, cta_counter, status, cycles);
  else
    dp_adamw_ag_kernel<__half><<<dp_grid(n_vec), 256, 0, stream>>>(
        p, f, world, rank, n_buckets, epoch, last, lo, n_vec, static_cast<const __half*>(grad),
        master, exp_avg, exp_avg_sq, decay_mask, grad_scale, lr, beta1, beta2, eps, weight_decay,
        bc1, bc2, cta_counter, status, cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int launch_peer_all_to_all(const void* src, void* const* dst_ptrs, int* const* flag_ptrs,
                           int world, int rank, int epoch, int outer, int rows, int row_bytes,
                           int64_t src_block_stride, int64_t src_outer_stride,
                           int64_t src_row_stride, int64_t dst_block_offset,
                           int64_t dst_outer_stride, int64_t dst_row_stride,
                           unsigned int* cta_counter, int* status, double wait_seconds,
                           cudaStream_t stream) {
  if (world < 1 || world > kDpMaxRanks || row_bytes % 16 != 0) return 1;
  const int64_t strides[6] = {src_block_stride, src_outer_stride, src_row_stride,
                              dst_block_offset, dst_outer_stride, dst_row_stride};
  for (int64_t v : strides)
    if (v % 16 != 0) return 2;   // byte strides must keep 16-byte alignment
  A2AParams p;
  p.src = src;
  for (int r = 0; r < kDpMaxRanks; ++r) {
    p.dst[r] = r < world ? dst_ptrs[r] : nullptr;
    p.flags[r] = r < world ? flag_ptrs[r] : nullptr;
  }
  p.world = world; p.rank = rank; p.epoch = epoch;
  p.outer = outer; p.rows = rows; p.row_vecs = row_bytes / 16;
  p.src_block_stride = src_block_stride / 16; p.src_outer_stride = src_outer_stride / 16;
  p.src_row_stride = src_row_stride / 16; p.dst_block_offset = dst_block_offset / 16;
  p.dst_outer_stride = dst_outer_stride / 16; p.dst_row_stride = dst_row_stride / 16;
  p.cta_counter = cta_counter; p.status = status; p.wait_cycles = dp_wait_cycles(wait_seconds);
  const int64_t total = static_cast<int64_t>(outer) * rows * p.row_vecs * world;
  count_launch();
  peer_all_to_all_kernel<<<dp_grid(total), 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int launch_vocab_embed_fwd(const int64_t* ids, const void* weight, void* const* out_ptrs,
                           int* const* flag_ptrs, int world, int rank, int epoch, int64_t tokens,
                           int hidden, int64_t vocab_lo, int64_t vocab_local, int scatter,
                           int64_t seq, unsigned int* cta_counter, int* status,
                           double wait_seconds, cudaStream_t stream) {
  if (world < 1 || world > kDpMaxRanks || hidden % 8 != 0) return 1;
  if (scatter == 1 && tokens % world != 0) return 1;
  if (scatter == 2 && (seq <= 0 || seq % world != 0 || tokens % seq != 0)) return 1;
  if (scatter < 0 || scatter > 2) return 1;
  VocabEmbedParams p;
  p.ids = ids; p.weight = weight;
  for (int r = 0; r < kDpMaxRanks; ++r) {
    p.out[r] = r < world ? out_ptrs[r] : nullptr;
    p.flags[r] = r < world ? flag_ptrs[r] : nullptr;
  }
  p.world = world; p.rank = rank; p.epoch = epoch; p.tokens = tokens;
  p.hidden_vecs = hidden / 8; p.vocab_lo = vocab_lo; p.vocab_local = vocab_local;
  p.scatter = scatter; p.seq = seq;
  p.cta_counter = cta_counter; p.status = status; p.wait_cycles = dp_wait_cycles(wait_seconds);
  int64_t blocks = (tokens + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  count_launch();
  vocab_embed_fwd_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace slapo
