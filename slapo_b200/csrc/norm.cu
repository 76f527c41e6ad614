// LayerNorm / RMSNorm, optionally fused with "bias + dropout + residual add"
// in front:   z = dropout(x + bias, p) + residual ;  y = norm(z) * gamma + beta
//
// One pass over HBM per direction: a row lives in registers (VPL vectors of 8
// per thread, WPR warps per row), statistics are two-pass in fp32, the
// dropout mask is regenerated from Philox in the backward, and the gamma /
// beta / bias gradients are accumulated in registers over all rows a CTA
// visits, written once per CTA to an fp32 scratch [grid, 3, cols] and summed
// by a small second kernel.
#include "common.cuh"
#include "kernels.h"

namespace slapo {

// Threads of a CTA are organised as RG row groups of WPR warps; each group
// normalises one row per iteration (VPL vectors of 8 values per thread).
// Several rows in flight per CTA keep enough loads outstanding to cover the
// HBM latency; group-local reductions use named barriers.
template <int WPR>
__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(32 * WPR) : "memory");
}

template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* red, int group, int wir) {
  v = warp_sum(v);
  if constexpr (WPR == 1) {
    return v;
  } else {
    const int lane = threadIdx.x & 31;
    if (lane == 0) red[group * WPR + wir] = v;
    group_sync<WPR>(group);
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) t += red[group * WPR + w];
    group_sync<WPR>(group);
    return t;
  }
}

template <typename T, int VPL, int WPR, int RG>
__global__ void __launch_bounds__(32 * WPR * RG, (VPL == 1 && WPR * RG == 16) ? 2 : 1) ln_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ residual,
    const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
    T* __restrict__ z, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
    int cols, float eps, float p, PhiloxArgs rng, int rms) {
  __shared__ float red[WPR * RG];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp / WPR, wir = warp % WPR;
  uint64_t seed = 0, offset = 0;
  if (p > 0.f) philox_unpack(rng, seed, offset);
  const float scale = dropout_scale(p);
  const float inv_cols = 1.f / static_cast<float>(cols);

  float gw[VPL][8], gb[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
    if (col < cols) {
      Vec8<T>::load(gamma + col, gw[i]);
      if (beta != nullptr) Vec8<T>::load(beta + col, gb[i]);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) gb[i][k] = 0.f;
      }
    }
  }

  for (int row0 = blockIdx.x * RG; row0 < rows; row0 += gridDim.x * RG) {
    const int row = row0 + group;
    const bool row_ok = row < rows;
    float v[VPL][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
      if (row_ok && col < cols) {
        const int64_t e = static_cast<int64_t>(row) * cols + col;
        Vec8<T>::load(x + e, v[i]);
        if (bias != nullptr) {
          float t[8];
          Vec8<T>::load(bias + col, t);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] += t[k];
        }
        if (p > 0.f) {
          bool keep[8];
          dropout_keep8(seed, offset, static_cast<uint64_t>(e), p, keep);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] = keep[k] ? v[i][k] * scale : 0.f;
        }
        if (residual != nullptr) {
          float t[8];
          Vec8<T>::load(residual + e, t);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] += t[k];
        }
        if (z != nullptr) {
          Vec8<T>::store(z + e, v[i]);
          // statistics must see exactly what the backward will re-read
          round_through<T>(v[i]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += v[i][k];
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] = 0.f;
      }
    }
    float mean = 0.f;
    if (!rms) mean = row_sum<WPR>(s, red, group, wir) * inv_cols;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
      if (col < cols) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { const float d = v[i][k] - mean; sq += d * d; }
      }
    }
    const float rstd = rsqrtf(row_sum<WPR>(sq, red, group, wir) * inv_cols + eps);
    if (row_ok) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
        if (col < cols) {
          float o[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] = (v[i][k] - mean) * rstd * gw[i][k] + gb[i][k];
          Vec8<T>::store(y + static_cast<int64_t>(row) * cols + col, o);
        }
      }
      if (lane == 0 && wir == 0) {
        mean_out[row] = mean;
        rstd_out[row] = rstd;
      }
    }
  }
}

template <typename T, int VPL, int WPR, int RG>
__global__ void __launch_bounds__(32 * WPR * RG, (VPL == 1 && WPR * RG == 16) ? 2 : 1) ln_bwd_kernel(
    const T* __restrict__ gy, const T* __restrict__ gz, const T* __restrict__ zin,
    const T* __restrict__ gamma, const float* __restrict__ mean_in,
    const float* __restrict__ rstd_in, T* __restrict__ dx, T* __restrict__ dres,
    float* __restrict__ partial, int rows, int cols, float p, PhiloxArgs rng, int rms,
    int want_dbias) {
  __shared__ float red[WPR * RG];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp / WPR, wir = warp % WPR;
  uint64_t seed = 0, offset = 0;
  if (p > 0.f) philox_unpack(rng, seed, offset);
  const float scale = dropout_scale(p);
  const float inv_cols = 1.f / static_cast<float>(cols);

  float gw[VPL][8], dgam[VPL][8], dbet[VPL][8], dbia[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
    if (col < cols) Vec8<T>::load(gamma + col, gw[i]);
#pragma unroll
    for (int k = 0; k < 8; ++k) { dgam[i][k] = 0.f; dbet[i][k] = 0.f; dbia[i][k] = 0.f; }
  }

  for (int row0 = blockIdx.x * RG; row0 < rows; row0 += gridDim.x * RG) {
    const int row = row0 + group;
    const bool row_ok = row < rows;
    const float mean = row_ok ? mean_in[row] : 0.f;
    const float rstd = row_ok ? rstd_in[row] : 0.f;
    float g[VPL][8], xh[VPL][8];
    uint4 gz_raw[VPL][sizeof(T) == 2 ? 1 : 2];  // fetched with the other operands, used after the reductions
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
      if (row_ok && col < cols) {
        const int64_t e = static_cast<int64_t>(row) * cols + col;
        Vec8<T>::load(gy + e, g[i]);
        Vec8<T>::load(zin + e, xh[i]);
        if (gz != nullptr) {
#pragma unroll
          for (int q = 0; q < (sizeof(T) == 2 ? 1 : 2); ++q)
            gz_raw[i][q] = reinterpret_cast<const uint4*>(gz + e)[q];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[i][k] = (xh[i][k] - mean) * rstd;
          dgam[i][k] += g[i][k] * xh[i][k];
          dbet[i][k] += g[i][k];
          g[i][k] *= gw[i][k];
          s1 += g[i][k];
          s2 += g[i][k] * xh[i][k];
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) { g[i][k] = 0.f; xh[i][k] = 0.f; }
      }
    }
    float m1 = 0.f;
    if (!rms) m1 = row_sum<WPR>(s1, red, group, wir) * inv_cols;
    const float m2 = row_sum<WPR>(s2, red, group, wir) * inv_cols;
    if (row_ok) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
        if (col < cols) {
          const int64_t e = static_cast<int64_t>(row) * cols + col;
          float d[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) d[k] = rstd * (g[i][k] - m1 - xh[i][k] * m2);
          if (gz != nullptr) {
            float t[8];
            Vec8<T>::load(reinterpret_cast<const T*>(gz_raw[i]), t);
#pragma unroll
            for (int k = 0; k < 8; ++k) d[k] += t[k];
          }
          if (dres != nullptr) Vec8<T>::store(dres + e, d);
          if (p > 0.f) {
            bool keep[8];
            dropout_keep8(seed, offset, static_cast<uint64_t>(e), p, keep);
#pragma unroll
            for (int k = 0; k < 8; ++k) d[k] = keep[k] ? d[k] * scale : 0.f;
          }
          if (want_dbias) {
#pragma unroll
            for (int k = 0; k < 8; ++k) dbia[i][k] += d[k];
          }
          Vec8<T>::store(dx + e, d);
        }
      }
    }
  }

  // one partial row per CTA: [grid][3][cols]; row groups are combined in
  // shared memory first
  float* out = partial + static_cast<int64_t>(blockIdx.x) * 3 * cols;
  if constexpr (RG > 1) {
    constexpr int kCap = 32 * WPR * VPL * 8;
    __shared__ float acc[3][kCap];
    for (int i = threadIdx.x; i < 3 * kCap; i += blockDim.x) (&acc[0][0])[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int c = (i * 32 * WPR + wir * 32 + lane) * 8 + k;
        atomicAdd(&acc[0][c], dgam[i][k]);
        atomicAdd(&acc[1][c], dbet[i][k]);
        atomicAdd(&acc[2][c], dbia[i][k]);
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      out[c] = acc[0][c];
      out[cols + c] = acc[1][c];
      out[2 * cols + c] = acc[2][c];
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int col = (i * 32 * WPR + wir * 32 + lane) * 8;
      if (col < cols) {
        Vec8<float>::store(out + col, dgam[i]);
        Vec8<float>::store(out + cols + col, dbet[i]);
        Vec8<float>::store(out + 2 * cols + col, dbia[i]);
      }
    }
  }
}

// Column sums of the per-CTA partials.  A 32 x 32 thread block owns 32 columns: threadIdx.y
// strides over the partial rows (coalesced 128-byte reads), shared memory combines the 32
// row groups - ~n_part / 32 dependent loads per thread instead of n_part.
template <typename T>
__global__ void __launch_bounds__(1024) ln_bwd_finalize_kernel(
    const float* __restrict__ partial, T* __restrict__ dgamma, T* __restrict__ dbeta,
    T* __restrict__ dbias, int n_part, int cols) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int which = blockIdx.y;  // 0 gamma, 1 beta, 2 bias
  T* dst = which == 0 ? dgamma : (which == 1 ? dbeta : dbias);
  if (dst == nullptr) return;
  float s = 0.f;
  if (c < cols) {
    for (int i = threadIdx.y; i < n_part; i += 32)
      s += partial[(static_cast<int64_t>(i) * 3 + which) * cols + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += red[y][threadIdx.x];
    if constexpr (sizeof(T) == 4) dst[c] = t;
    else dst[c] = static_cast<T>(t);
  }
}

// ------------------------------------------------------------------------ //
struct LnShape { int vpl; int wpr; int rg; };

static LnShape pick_shape(int cols) {
  const int vecs = cols / 8;
  if (vecs <= 32) return {1, 1, 4};
  // for 1024 columns one warp per row (4 vectors per lane) and two warps per row were
  // measured slower (fwd 341 / 199 us, bwd 457 / 309 us on 65536 rows) than four warps per row
  // with four row groups per CTA (129 / 264 us): registers, not barriers, limit the latter
  if (vecs <= 128) return {1, 4, 4};
  if (vecs <= 256) return {2, 4, 4};
  if (vecs <= 512) return {1, 16, 1};
  if (vecs <= 1024) return {2, 16, 1};
  return {4, 16, 1};
}

static int ln_grid(int rows, int cols, int ctas_per_sm) {
  const LnShape s = pick_shape(cols);
  const int want = (rows + s.rg - 1) / s.rg;
  const int cap = sm_count() * ctas_per_sm;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

int ln_bwd_grid(int rows, int cols) {
  const LnShape s = pick_shape(cols);
  return ln_grid(rows, cols, s.wpr * s.rg >= 16 ? 2 : 8);
}

#define LN_SHAPE_SWITCH(s, ...)                                                     \
  if (s.wpr == 1) {                                                          \
    constexpr int WPR = 1, RG = 4, VPL = 1;                                         \
    __VA_ARGS__;                                                                    \
  } else if (s.wpr == 4) {                                                          \
    constexpr int WPR = 4, RG = 4;                                                  \
    if (s.vpl == 1) { constexpr int VPL = 1; __VA_ARGS__; }                         \
    else { constexpr int VPL = 2; __VA_ARGS__; }                                    \
  } else {                                                                          \
    constexpr int WPR = 16, RG = 1;                                                 \
    if (s.vpl == 1) { constexpr int VPL = 1; __VA_ARGS__; }                         \
    else if (s.vpl == 2) { constexpr int VPL = 2; __VA_ARGS__; }                    \
    else { constexpr int VPL = 4; __VA_ARGS__; }                                    \
  }

#define DISPATCH_DTYPE(dtype, ...)                                   \
  switch (dtype) {                                                   \
    case 0: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    case 1: { using T = __half; __VA_ARGS__; break; }                \
    default: { using T = float; __VA_ARGS__; break; }                \
  }

void launch_ln_fwd(const void* x, const void* bias, const void* residual, const void* gamma,
                   const void* beta, void* y, void* z, float* mean, float* rstd, int rows,
                   int cols, float eps, float p, PhiloxArgs rng, int rms, int dtype,
                   cudaStream_t stream) {
  if (rows == 0) return;
  const LnShape s = pick_shape(cols);
  const int grid = ln_grid(rows, cols, s.wpr * s.rg >= 16 ? 2 : 16);
  count_launch();
  DISPATCH_DTYPE(dtype, LN_SHAPE_SWITCH(s, (ln_fwd_kernel<T, VPL, WPR, RG>
      <<<grid, 32 * WPR * RG, 0, stream>>>(
          static_cast<const T*>(x), static_cast<const T*>(bias), static_cast<const T*>(residual),
          static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y),
          static_cast<T*>(z), mean, rstd, rows, cols, eps, p, rng, rms))));
}

void launch_ln_bwd(const void* gy, const void* gz, const void* zin, const void* gamma,
                   const float* mean, const float* rstd, void* dx, void* dres, void* dgamma,
                   void* dbeta, void* dbias, float* partial, int rows, int cols, float p,
                   PhiloxArgs rng, int rms, int dtype, cudaStream_t stream) {
  if (rows == 0) return;
  const LnShape s = pick_shape(cols);
  const int grid = ln_bwd_grid(rows, cols);
  const int want_dbias = dbias != nullptr;
  count_launch(2);
  DISPATCH_DTYPE(dtype, LN_SHAPE_SWITCH(s, (ln_bwd_kernel<T, VPL, WPR, RG>
      <<<grid, 32 * WPR * RG, 0, stream>>>(
          static_cast<const T*>(gy), static_cast<const T*>(gz), static_cast<const T*>(zin),
          static_cast<const T*>(gamma), mean, rstd, static_cast<T*>(dx), static_cast<T*>(dres),
          partial, rows, cols, p, rng, rms, want_dbias))));
  dim3 fgrid((cols + 31) / 32, 3);
  DISPATCH_DTYPE(dtype, (ln_bwd_finalize_kernel<T><<<fgrid, dim3(32, 32), 0, stream>>>(
      partial, static_cast<T*>(dgamma), static_cast<T*>(dbeta), static_cast<T*>(dbias), grid,
      cols)));
}

}  // namespace slapo
