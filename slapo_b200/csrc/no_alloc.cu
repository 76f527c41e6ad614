// Allocation-free C entry point for the bias + activation backward; the
// contract (limits, set-up, concurrency) is spelled out in no_alloc.h.
#include "no_alloc.h"

#include <mutex>
#include <stdio.h>

#include "kernels.h"

namespace {

// Per-chunk column sums of the bias gradient, [chunks, cols] fp32.  One copy
// of this array exists on every device that loads the library image.
static __device__ __align__(256) float g_colsum_scratch[SLAPO_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

int fail(int code, char* err, int err_len, const char* fmt, long a = 0, long b = 0, long c = 0) {
  if (err != nullptr && err_len > 0) snprintf(err, static_cast<size_t>(err_len), fmt, a, b, c);
  return code;
}

// Device address of the scratch array on the current device; looked up once per
// device.  Returns nullptr (and the CUDA error in *rc) on failure.
float* scratch_for_current_device(cudaError_t* rc) {
  int dev = -1;
  *rc = cudaGetDevice(&dev);
  if (*rc != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    *rc = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    *rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_scratch);
    if (*rc != cudaSuccess) return nullptr;
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int slapo_bias_act_bwd_noalloc(const void* dy, const void* x, const void* bias,
                                          void* dx, void* dbias, int rows, int cols, int act,
                                          int dtype, cudaStream_t stream, char* err,
                                          int err_len) {
  if (dy == nullptr || x == nullptr || dx == nullptr)
    return fail(SLAPO_NOALLOC_E_ARGUMENT, err, err_len, "dy, x and dx must not be NULL");
  if (rows < 0 || cols <= 0 || cols % 8 != 0)
    return fail(SLAPO_NOALLOC_E_ARGUMENT, err, err_len,
                "rows=%ld cols=%ld: rows must be >= 0 and cols a positive multiple of 8", rows,
                cols);
  if (dtype < 0 || dtype > 2 || act < 0 || act > 2)
    return fail(SLAPO_NOALLOC_E_ARGUMENT, err, err_len, "dtype=%ld act=%ld: codes are 0..2",
                dtype, act);
  if (cols > SLAPO_NOALLOC_MAX_COLS)
    return fail(SLAPO_NOALLOC_E_TOO_LARGE, err, err_len,
                "cols=%ld exceeds the maximum of %ld for the allocation-free entry point", cols,
                SLAPO_NOALLOC_MAX_COLS);
  if (rows == 0) return SLAPO_NOALLOC_OK;

  float* scratch = nullptr;
  if (dbias != nullptr) {
    const long need = static_cast<long>(slapo::colsum_chunks(rows, cols)) * cols;
    if (need > SLAPO_NOALLOC_SCRATCH_FLOATS)
      return fail(SLAPO_NOALLOC_E_TOO_LARGE, err, err_len,
                  "rows=%ld cols=%ld need %ld scratch floats; the static scratch holds fewer",
                  rows, cols, need);
    cudaError_t rc = cudaSuccess;
    scratch = scratch_for_current_device(&rc);
    if (scratch == nullptr)
      return fail(SLAPO_NOALLOC_E_CUDA, err, err_len,
                  "looking up the scratch array failed with CUDA error %ld", static_cast<long>(rc));
  }
  // only an error that THIS launch raised is reported: an error that was already pending on the
  // thread (someone else's failed call) is neither consumed nor blamed on this one
  const cudaError_t before = cudaPeekAtLastError();
  slapo::launch_bias_act_bwd(dy, x, bias, dx, dbias, scratch, rows, cols, act, dtype, stream);
  const cudaError_t after = cudaPeekAtLastError();
  if (after != cudaSuccess && after != before)
    return fail(SLAPO_NOALLOC_E_CUDA, err, err_len, "kernel launch failed with CUDA error %ld",
                static_cast<long>(after));
  return SLAPO_NOALLOC_OK;
}

extern "C" long slapo_bias_act_bwd_noalloc_scratch_floats(int rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<long>(slapo::colsum_chunks(rows, cols)) * cols;
}
