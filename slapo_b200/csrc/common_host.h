// Launchers that take a PhiloxArgs by value need its full definition; it is
// kept free of device-only constructs so that host compilers can include it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef __CUDACC__
namespace slapo {
struct PhiloxArgs {
  uint64_t seed;
  uint64_t offset;
  const int64_t* seed_ptr;
  const int64_t* offset_ptr;
  uint32_t offset_intragraph;
  int captured;
};
}  // namespace slapo
#endif

namespace slapo {
void launch_bias_dropout_add_fwd(const void* x, const void* bias, const void* residual, void* y,
                                 int64_t rows, int cols, float p, PhiloxArgs rng, int dtype,
                                 cudaStream_t stream);
void launch_bias_dropout_add_bwd(const void* dy, void* dx, void* dbias, float* partial, int rows,
                                 int cols, float p, PhiloxArgs rng, int dtype,
                                 cudaStream_t stream);
void launch_ln_fwd(const void* x, const void* bias, const void* residual, const void* gamma,
                   const void* beta, void* y, void* z, float* mean, float* rstd, int rows,
                   int cols, float eps, float p, PhiloxArgs rng, int rms, int dtype,
                   cudaStream_t stream);
void launch_ln_bwd(const void* gy, const void* gz, const void* zin, const void* gamma,
                   const float* mean, const float* rstd, void* dx, void* dres, void* dgamma,
                   void* dbeta, void* dbias, float* partial, int rows, int cols, float p,
                   PhiloxArgs rng, int rms, int dtype, cudaStream_t stream);
}  // namespace slapo

namespace slapo {
// Flash attention on [B, S, H, D] tensors (D contiguous, a multiple of 8 up to 128);
// *_strides = element strides of (B, S, H).  Return 0 on success.
int launch_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                     const float* kbias, const float* rel, int B, int H, int Sq, int Sk, int D,
                     const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                     float scale, int causal, float p_drop, PhiloxArgs rng, bool bf16, int* status,
                     cudaStream_t stream);
int launch_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                     const float* lse, float* delta, float* dq_accum, int64_t dq_slice_stride,
                     void* dk, void* dv, int64_t dkv_row_stride, const float* kbias, const float* rel, float* drel,
                     int B, int H, int Sq, int Sk, int D, const int64_t* q_strides, const int64_t* k_strides,
                     const int64_t* v_strides, float scale, int causal, float p_drop,
                     PhiloxArgs rng, bool bf16, int* status, cudaStream_t stream);
void launch_flash_dq_convert(const float* acc, void* out, int64_t rows, int D,
                             int64_t out_row_stride, bool bf16, int n_slices, int64_t slice_stride,
                             int Sq, int Sk, int H, int causal, cudaStream_t stream);
void launch_flash_dropout_mask(uint8_t* mask, int B, int H, int Sq, int Sk, float p_drop,
                               PhiloxArgs rng, cudaStream_t stream);
}  // namespace slapo
