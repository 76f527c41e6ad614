// Cross-entropy over a (possibly vocabulary-sharded) logit matrix, and the
// squared-norm reduction used for gradient clipping.
//
// Cross entropy is split so that the same kernels serve one GPU and a
// tensor-parallel group whose ranks each hold a vocabulary slice
// [vocab_start, vocab_start + V):
//   ce_stats   one CTA per token row, one streaming pass over the row:
//              stats[row] = (max, sum exp(x - max), logit of the target if it
//              lies in this slice else 0).  Rows whose label is the ignore
//              index are not read at all.
//   (group)    the caller combines the three numbers over the group
//              (MAX / rescaled SUM / SUM) - nothing to do on one GPU.
//   ce_grad    grad[row, :] = (exp(x - lse) - onehot(target)) * coef[row],
//              written in the logits' dtype; ignored rows get zeros.
#include "common.cuh"
#include "kernels.h"

namespace slapo {

template <typename T>
__global__ void __launch_bounds__(256) ce_stats_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ stats,
    int rows, int cols, int64_t row_stride, int vocab_start, int64_t ignore_index) {
  __shared__ float red_m[8], red_s[8];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int64_t label = labels[row];
  float* out = stats + static_cast<int64_t>(row) * 3;
  if (label == ignore_index) {
    if (threadIdx.x == 0) { out[0] = -INFINITY; out[1] = 0.f; out[2] = 0.f; }
    return;
  }
  const T* x = logits + static_cast<int64_t>(row) * row_stride;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    float v[8];
    Vec8<T>::load(x + c, v);
    float cm = v[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) cm = fmaxf(cm, v[k]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += __expf(v[k] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  // combine (m, s) over the CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float fm = red_m[0], fs = red_s[0];
    for (int w = 1; w < 8; ++w) {
      const float nm = fmaxf(fm, red_m[w]);
      fs = (fm == -INFINITY ? 0.f : fs * __expf(fm - nm)) +
           (red_m[w] == -INFINITY ? 0.f : red_s[w] * __expf(red_m[w] - nm));
      fm = nm;
    }
    const int64_t local = label - vocab_start;
    float picked = 0.f;
    if (local >= 0 && local < cols) picked = static_cast<float>(x[local]);
    out[0] = fm; out[1] = fs; out[2] = picked;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ce_grad_kernel(
    const T* __restrict__ logits, const int64_t* __restrict__ labels,
    const float* __restrict__ lse, const float* __restrict__ coef, T* __restrict__ grad, int rows,
    int cols, int64_t row_stride, int vocab_start, int64_t ignore_index) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int64_t label = labels[row];
  T* g = grad + static_cast<int64_t>(row) * row_stride;
  if (label == ignore_index) {
    const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) Vec8<T>::store(g + c, z);
    return;
  }
  const T* x = logits + static_cast<int64_t>(row) * row_stride;
  const float l = lse[row], w = coef[row];
  const int local = static_cast<int>(label - vocab_start);
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    float v[8];
    Vec8<T>::load(x + c, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(v[k] - l);
      if (c + k == local) p -= 1.f;
      v[k] = p * w;
    }
    Vec8<T>::store(g + c, v);
  }
}

// sum of squares of a flat low-precision buffer, split by an optional byte
// mask: out[0] += sum over mask == 0, out[1] += sum over mask == 1; other values are skipped.
template <typename T>
__global__ void __launch_bounds__(256) sq_norm_kernel(const T* __restrict__ x,
                                                      const uint8_t* __restrict__ mask,
                                                      float* __restrict__ out, int64_t n_vec) {
  __shared__ float red[2][8];
  float a0 = 0.f, a1 = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += stride) {
    float v[8];
    Vec8<T>::load(x + i * 8, v);
    if (mask != nullptr) {
      const uint2 mk = *reinterpret_cast<const uint2*>(mask + i * 8);
      const uint8_t* mb = reinterpret_cast<const uint8_t*>(&mk);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (mb[k] == 1) a1 += v[k] * v[k];
        else if (mb[k] == 0) a0 += v[k] * v[k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) a0 += v[k] * v[k];
    }
  }
  a0 = warp_sum(a0);
  a1 = warp_sum(a1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red[0][warp] = a0; red[1][warp] = a1; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s0 = 0.f, s1 = 0.f;
    for (int w = 0; w < 8; ++w) { s0 += red[0][w]; s1 += red[1][w]; }
    atomicAdd(out, s0);
    atomicAdd(out + 1, s1);
  }
}

#define DISPATCH_DTYPE(dtype, ...)                                   \
  switch (dtype) {                                                   \
    case 0: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    case 1: { using T = __half; __VA_ARGS__; break; }                \
    default: { using T = float; __VA_ARGS__; break; }                \
  }

void launch_ce_stats(const void* logits, const int64_t* labels, float* stats, int rows, int cols,
                     int64_t row_stride, int vocab_start, int64_t ignore_index, int dtype,
                     cudaStream_t stream) {
  if (rows == 0) return;
  count_launch();
  DISPATCH_DTYPE(dtype, (ce_stats_kernel<T><<<rows, 256, 0, stream>>>(
      static_cast<const T*>(logits), labels, stats, rows, cols, row_stride, vocab_start,
      ignore_index)));
}

void launch_ce_grad(const void* logits, const int64_t* labels, const float* lse,
                    const float* coef, void* grad, int rows, int cols, int64_t row_stride,
                    int vocab_start, int64_t ignore_index, int dtype, cudaStream_t stream) {
  if (rows == 0) return;
  count_launch();
  DISPATCH_DTYPE(dtype, (ce_grad_kernel<T><<<rows, 256, 0, stream>>>(
      static_cast<const T*>(logits), labels, lse, coef, static_cast<T*>(grad), rows, cols,
      row_stride, vocab_start, ignore_index)));
}

void launch_sq_norm(const void* x, const uint8_t* mask, float* out2, int64_t n, int dtype,
                    cudaStream_t stream) {
  const int64_t n_vec = n / 8;
  if (n_vec == 0) return;
  int64_t blocks = (n_vec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  count_launch();
  DISPATCH_DTYPE(dtype, (sq_norm_kernel<T><<<static_cast<int>(blocks), 256, 0, stream>>>(
      static_cast<const T*>(x), mask, out2, n_vec)));
}

}  // namespace slapo
