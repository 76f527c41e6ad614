// Fused element-wise kernels (HBM-bound, one pass each):
//   bias_act          y = act(x + bias)                       fwd / bwd (+ reduced dbias)
//   bias_dropout_add  y = dropout(x + bias, p) + residual     fwd / bwd (+ reduced dbias)
//   fused_adamw       AdamW on flat fp32 master weights, writes the low-precision copy
// Dropout masks are regenerated from Philox (seed, offset, element index): no
// mask tensor exists.  Bias gradients are reduced in two stages through a
// small fp32 scratch buffer [row_chunks, cols] supplied by the caller.
#include "common.cuh"
#include "kernels.h"

#include <atomic>

namespace slapo {

static std::atomic<int64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// ------------------------------------------------------------------------ //
// Four independent 16-byte loads per thread are issued before any of them is used: with
// 2048 resident threads per SM a single load each leaves too few bytes in flight to cover the
// HBM latency at full bandwidth.
template <typename T>
__global__ void __launch_bounds__(256) bias_act_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, int64_t n_vec,
    int cols, int act) {
  constexpr int kUnroll = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int vpr = cols / kVec;  // vectors per row
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // column (in vectors) of the first vector and its advance per step, kept in 32 bits
  int cv = static_cast<int>(i % vpr);
  const int step = static_cast<int>(stride % vpr);
  for (; i + (kUnroll - 1) * stride < n_vec; i += kUnroll * stride) {
    float v[kUnroll][8];
    int cvs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Vec8<T>::load(x + (i + u * stride) * kVec, v[u]);
      cvs[u] = cv;
      cv += step;
      if (cv >= vpr) cv -= vpr;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (bias != nullptr) {
        float b[8];
        Vec8<T>::load(bias + cvs[u] * kVec, b);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[u][k] += b[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[u][k] = act_fwd(v[u][k], act);
      Vec8<T>::store(y + (i + u * stride) * kVec, v[u]);
    }
  }
  for (; i < n_vec; i += stride) {
    float v[8];
    Vec8<T>::load(x + i * kVec, v);
    if (bias != nullptr) {
      float b[8];
      Vec8<T>::load(bias + cv * kVec, b);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += b[k];
    }
    cv += step;
    if (cv >= vpr) cv -= vpr;
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = act_fwd(v[k], act);
    Vec8<T>::store(y + i * kVec, v);
  }
}

// Column-slab layout shared by the backward kernels: a CTA of 8 warps covers
// 256 columns (lane -> 8 columns) and a chunk of rows (warp w takes rows
// w, w+8, ...).  Per-thread partial column sums are combined across the 8
// warps in shared memory and written to partial[blockIdx.y][col].
__device__ __forceinline__ void slab_reduce_store(float acc[8], float* partial, int cols,
                                                  int col, bool col_ok) {
  __shared__ float red[8][256 + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < 8; ++k) red[warp][lane * 8 + k] = acc[k];
  __syncthreads();
  if (warp == 0 && col_ok) {
    float s[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[w][lane * 8 + k];
      s[k] = t;
    }
    Vec8<float>::store(partial + static_cast<int64_t>(blockIdx.y) * cols + col, s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bias_act_bwd_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ bias,
    T* __restrict__ dx, float* __restrict__ partial, int rows, int cols, int rows_per_chunk,
    int act) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 256 + lane * 8;
  const bool col_ok = col + 8 <= cols;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col_ok) {
    if (bias != nullptr) Vec8<T>::load(bias + col, b);
    const int r0 = blockIdx.y * rows_per_chunk;
    const int r1 = min(rows, r0 + rows_per_chunk);
#pragma unroll 4
    for (int r = r0 + warp; r < r1; r += 8) {
      const int64_t e = static_cast<int64_t>(r) * cols + col;
      float g[8], v[8];
      Vec8<T>::load(dy + e, g);
      Vec8<T>::load(x + e, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        g[k] *= act_grad(v[k] + b[k], act);
        acc[k] += g[k];
      }
      Vec8<T>::store(dx + e, g);
    }
  }
  if (partial != nullptr) slab_reduce_store(acc, partial, cols, col, col_ok);
}

// Column sums of a [rows, cols] matrix (the bias gradient of a plain linear layer): same slab
// decomposition as above, reading only.
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ x,
                                                     float* __restrict__ partial, int rows,
                                                     int cols, int64_t row_stride,
                                                     int rows_per_chunk) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 256 + lane * 8;
  const bool col_ok = col + 8 <= cols;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col_ok) {
    const int r0 = blockIdx.y * rows_per_chunk;
    const int r1 = min(rows, r0 + rows_per_chunk);
#pragma unroll 4
    for (int r = r0 + warp; r < r1; r += 8) {
      float g[8];
      Vec8<T>::load(x + static_cast<int64_t>(r) * row_stride + col, g);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g[k];
    }
  }
  slab_reduce_store(acc, partial, cols, col, col_ok);
}

// 32 x 32 threads per 32 columns: threadIdx.y strides over the chunks (see ln_bwd_finalize).
template <typename T>
__global__ void __launch_bounds__(1024) colsum_finalize_kernel(
    const float* __restrict__ partial, T* __restrict__ out, int chunks, int cols) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols) {
    for (int i = threadIdx.y; i < chunks; i += 32) s += partial[static_cast<int64_t>(i) * cols + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += red[y][threadIdx.x];
    if constexpr (sizeof(T) == 4) out[c] = t;
    else out[c] = static_cast<T>(t);
  }
}

// ------------------------------------------------------------------------ //
template <typename T>
__global__ void __launch_bounds__(256) bias_dropout_add_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ residual,
    T* __restrict__ y, int64_t n_vec, int cols, float p, PhiloxArgs rng) {
  uint64_t seed, offset;
  philox_unpack(rng, seed, offset);
  const float scale = dropout_scale(p);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += stride) {
    const int64_t e = i * kVec;
    float v[8], t[8];
    bool keep[8];
    Vec8<T>::load(x + e, v);
    if (bias != nullptr) {
      Vec8<T>::load(bias + (e % cols), t);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += t[k];
    }
    dropout_keep8(seed, offset, static_cast<uint64_t>(e), p, keep);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = keep[k] ? v[k] * scale : 0.f;
    if (residual != nullptr) {
      Vec8<T>::load(residual + e, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += t[k];
    }
    Vec8<T>::store(y + e, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bias_dropout_add_bwd_kernel(
    const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ partial, int rows,
    int cols, int rows_per_chunk, float p, PhiloxArgs rng) {
  uint64_t seed, offset;
  philox_unpack(rng, seed, offset);
  const float scale = dropout_scale(p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 256 + lane * 8;
  const bool col_ok = col + 8 <= cols;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col_ok) {
    const int r0 = blockIdx.y * rows_per_chunk;
    const int r1 = min(rows, r0 + rows_per_chunk);
    for (int r = r0 + warp; r < r1; r += 8) {
      const int64_t e = static_cast<int64_t>(r) * cols + col;
      float g[8];
      bool keep[8];
      Vec8<T>::load(dy + e, g);
      dropout_keep8(seed, offset, static_cast<uint64_t>(e), p, keep);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        g[k] = keep[k] ? g[k] * scale : 0.f;
        acc[k] += g[k];
      }
      Vec8<T>::store(dx + e, g);
    }
  }
  if (partial != nullptr) slab_reduce_store(acc, partial, cols, col, col_ok);
}

// ------------------------------------------------------------------------ //
template <typename T>
__global__ void __launch_bounds__(256) fused_adamw_kernel(
    T* __restrict__ param, const T* __restrict__ grad, float* __restrict__ master,
    float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
    const uint8_t* __restrict__ decay_mask, const float* __restrict__ grad_scale, int64_t n_vec,
    float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
    const float* __restrict__ hyper) {
  // hyper = {lr, bias correction 1, bias correction 2} in device memory: the values that change
  // from step to step, so that a captured CUDA graph of the step stays valid
  if (hyper != nullptr) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }
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
    Vec8<T>::store(param + e, w);
  }
}

// ------------------------------------------------------------------------ //
static inline int flat_grid(int64_t n_vec) {
  int64_t blocks = (n_vec + 255) / 256;
  int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

int colsum_chunks(int rows, int cols) {
  const int slabs = (cols + 255) / 256;
  int chunks = (sm_count() * 8 + slabs - 1) / slabs;
  const int max_chunks = (rows + 7) / 8;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  return chunks;
}

#define DISPATCH_DTYPE(dtype, ...)                                   \
  switch (dtype) {                                                   \
    case 0: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    case 1: { using T = __half; __VA_ARGS__; break; }                \
    default: { using T = float; __VA_ARGS__; break; }                \
  }

void launch_bias_act_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols,
                         int act, int dtype, cudaStream_t stream) {
  const int64_t n_vec = rows * cols / kVec;
  if (n_vec == 0) return;
  count_launch();
  DISPATCH_DTYPE(dtype, (bias_act_fwd_kernel<T><<<flat_grid(n_vec), 256, 0, stream>>>(
      static_cast<const T*>(x), static_cast<const T*>(bias), static_cast<T*>(y), n_vec, cols, act)));
}

void launch_colsum_finalize(const float* partial, void* out, int chunks, int cols, int dtype,
                            cudaStream_t stream) {
  count_launch();
  DISPATCH_DTYPE(dtype, (colsum_finalize_kernel<T><<<(cols + 31) / 32, dim3(32, 32), 0, stream>>>(
      partial, static_cast<T*>(out), chunks, cols)));
}

void launch_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, void* dbias,
                         float* partial, int rows, int cols, int act, int dtype,
                         cudaStream_t stream) {
  if (rows == 0) return;
  const int chunks = colsum_chunks(rows, cols);
  const int rows_per_chunk = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 255) / 256, chunks);
  float* part = dbias != nullptr ? partial : nullptr;
  count_launch();
  DISPATCH_DTYPE(dtype, (bias_act_bwd_kernel<T><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(bias),
      static_cast<T*>(dx), part, rows, cols, rows_per_chunk, act)));
  if (dbias != nullptr) launch_colsum_finalize(partial, dbias, chunks, cols, dtype, stream);
}

void launch_colsum(const void* x, void* out, float* partial, int rows, int cols,
                   int64_t row_stride, int dtype, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return;
  const int chunks = colsum_chunks(rows, cols);
  const int rows_per_chunk = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 255) / 256, chunks);
  count_launch();
  DISPATCH_DTYPE(dtype, (colsum_kernel<T><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(x), partial, rows, cols, row_stride, rows_per_chunk)));
  launch_colsum_finalize(partial, out, chunks, cols, dtype, stream);
}

void launch_bias_dropout_add_fwd(const void* x, const void* bias, const void* residual, void* y,
                                 int64_t rows, int cols, float p, PhiloxArgs rng, int dtype,
                                 cudaStream_t stream) {
  const int64_t n_vec = rows * cols / kVec;
  if (n_vec == 0) return;
  count_launch();
  DISPATCH_DTYPE(dtype, (bias_dropout_add_fwd_kernel<T><<<flat_grid(n_vec), 256, 0, stream>>>(
      static_cast<const T*>(x), static_cast<const T*>(bias), static_cast<const T*>(residual),
      static_cast<T*>(y), n_vec, cols, p, rng)));
}

void launch_bias_dropout_add_bwd(const void* dy, void* dx, void* dbias, float* partial, int rows,
                                 int cols, float p, PhiloxArgs rng, int dtype,
                                 cudaStream_t stream) {
  if (rows == 0) return;
  const int chunks = colsum_chunks(rows, cols);
  const int rows_per_chunk = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 255) / 256, chunks);
  float* part = dbias != nullptr ? partial : nullptr;
  count_launch();
  DISPATCH_DTYPE(dtype, (bias_dropout_add_bwd_kernel<T><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(dy), static_cast<T*>(dx), part, rows, cols, rows_per_chunk, p, rng)));
  if (dbias != nullptr) launch_colsum_finalize(partial, dbias, chunks, cols, dtype, stream);
}

void launch_fused_adamw(void* param, const void* grad, float* master, float* exp_avg,
                        float* exp_avg_sq, const uint8_t* decay_mask, const float* grad_scale,
                        int64_t n, float lr, float beta1, float beta2, float eps,
                        float weight_decay, float bc1, float bc2, int dtype,
                        cudaStream_t stream, const float* hyper) {
  const int64_t n_vec = n / kVec;
  if (n_vec == 0) return;
  count_launch();
  DISPATCH_DTYPE(dtype, (fused_adamw_kernel<T><<<flat_grid(n_vec), 256, 0, stream>>>(
      static_cast<T*>(param), static_cast<const T*>(grad), master, exp_avg, exp_avg_sq, decay_mask,
      grad_scale, n_vec, lr, beta1, beta2, eps, weight_decay, bc1, bc2, hyper)));
}

}  // namespace slapo
