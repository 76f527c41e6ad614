// Shared device helpers: 8-wide vector access for bf16/fp16/fp32, warp
// reductions, Philox4x32-10 with an (optionally device-resident) seed/offset.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace slapo {

constexpr int kVec = 8;  // elements per thread access (16 bytes of 16-bit data)

// ---------------------------------------------------------------------------
// Philox state handed over from the host.  In eager mode `seed`/`offset` hold
// values; under CUDA-graph capture they are read through the pointers, which
// the framework's generator refreshes before every replay.
struct PhiloxArgs {
  uint64_t seed;
  uint64_t offset;
  const int64_t* seed_ptr;
  const int64_t* offset_ptr;
  uint32_t offset_intragraph;
  int captured;
};

__device__ __forceinline__ void philox_unpack(const PhiloxArgs& a, uint64_t& seed,
                                              uint64_t& offset) {
  if (a.captured) {
    seed = static_cast<uint64_t>(*a.seed_ptr);
    offset = static_cast<uint64_t>(*a.offset_ptr) + a.offset_intragraph;
  } else {
    seed = a.seed;
    offset = a.offset;
  }
}

__device__ __forceinline__ uint2 mulhilo32(uint32_t a, uint32_t b) {
  uint64_t p = static_cast<uint64_t>(a) * b;
  return make_uint2(static_cast<uint32_t>(p), static_cast<uint32_t>(p >> 32));
}

// Philox4x32-10 of the 128-bit counter {offset, index}: a pure function of
// (seed, offset, index), so forward and backward regenerate the same bits
// whatever the thread mapping.
__device__ __forceinline__ uint4 philox4x32(uint64_t seed, uint64_t offset, uint64_t index) {
  uint4 c = make_uint4(static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32),
                       static_cast<uint32_t>(index), static_cast<uint32_t>(index >> 32));
  uint2 k = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint2 m0 = mulhilo32(0xD2511F53u, c.x);
    uint2 m1 = mulhilo32(0xCD9E8D57u, c.z);
    c = make_uint4(m1.y ^ c.y ^ k.x, m1.x, m0.y ^ c.w ^ k.y, m0.x);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

// Cheaper variant for attention-probability dropout: 7 rounds and 16-bit
// draws, so one call serves 8 consecutive keys of one query row.  Bit k of
// the result is set when key k is kept (draw >= p * 65536).
__device__ __forceinline__ uint32_t philox_keep8_u16(uint64_t seed, uint64_t offset,
                                                     uint64_t index, uint32_t thr16) {
  uint4 c = make_uint4(static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32),
                       static_cast<uint32_t>(index), static_cast<uint32_t>(index >> 32));
  uint2 k = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    uint2 m0 = mulhilo32(0xD2511F53u, c.x);
    uint2 m1 = mulhilo32(0xCD9E8D57u, c.z);
    c = make_uint4(m1.y ^ c.y ^ k.x, m1.x, m0.y ^ c.w ^ k.y, m0.x);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  uint32_t bits = 0;
  bits |= ((c.x & 0xffffu) >= thr16) << 0;
  bits |= ((c.x >> 16) >= thr16) << 1;
  bits |= ((c.y & 0xffffu) >= thr16) << 2;
  bits |= ((c.y >> 16) >= thr16) << 3;
  bits |= ((c.z & 0xffffu) >= thr16) << 4;
  bits |= ((c.z >> 16) >= thr16) << 5;
  bits |= ((c.w & 0xffffu) >= thr16) << 6;
  bits |= ((c.w >> 16) >= thr16) << 7;
  return bits;
}

// keep-mask bits for 8 consecutive elements starting at element index e0
// (e0 a multiple of 8): element e uses word (e % 4) of philox(index = e / 4).
__device__ __forceinline__ void dropout_keep8(uint64_t seed, uint64_t offset, uint64_t e0,
                                              float p, bool keep[8]) {
  uint4 r0 = philox4x32(seed, offset, e0 >> 2);
  uint4 r1 = philox4x32(seed, offset, (e0 >> 2) + 1);
  const uint32_t thr = static_cast<uint32_t>(fminf(p, 1.f) * 4294967295.0f);
  keep[0] = r0.x >= thr; keep[1] = r0.y >= thr; keep[2] = r0.z >= thr; keep[3] = r0.w >= thr;
  keep[4] = r1.x >= thr; keep[5] = r1.y >= thr; keep[6] = r1.z >= thr; keep[7] = r1.w >= thr;
}

// ---------------------------------------------------------------------------
template <typename T> struct Vec8;

template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float v[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float v[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float v[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float v[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float v[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float v[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// round fp32 values to the storage type and back (what a later re-read sees)
template <typename T>
__device__ __forceinline__ void round_through(float v[8]) {
  if constexpr (sizeof(T) == 2) {
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = static_cast<float>(static_cast<T>(v[k]));
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// activation codes shared with the Python side: 0 = GeLU (erf), 1 = GeLU (tanh), 2 = ReLU
__device__ __forceinline__ float act_fwd(float x, int act) {
  if (act == 0) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  if (act == 1) {
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return fmaxf(x, 0.f);
}

__device__ __forceinline__ float act_grad(float x, int act) {
  if (act == 0) {
    float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return cdf + x * pdf;
  }
  if (act == 1) {
    float x2 = x * x;
    float u = 0.7978845608028654f * (x + 0.044715f * x * x2);
    float t = tanhf(u);
    float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
  }
  return x > 0.f ? 1.f : 0.f;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace slapo
