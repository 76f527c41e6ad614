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

// Attention-probability dropout: one 7-round Philox call decides 16
// consecutive keys of one query row.  Each of the 16 result bytes yields a
// 7-bit draw; a key is kept when draw >= thr7, so the dropout probability is
// quantised to thr7 / 128.  ``add4`` = (128 - thr7) * 0x01010101: adding it to
// the draws (byte lanes cannot carry into each other: 127 + 128 = 255) leaves
// bit 7 of byte j of word w set exactly when key 4 w + j is kept.
__device__ __forceinline__ uint4 philox_keep16(uint64_t seed, uint64_t offset, uint64_t index,
                                               uint32_t add4) {
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
  c.x = (c.x & 0x7f7f7f7fu) + add4;
  c.y = (c.y & 0x7f7f7f7fu) + add4;
  c.z = (c.z & 0x7f7f7f7fu) + add4;
  c.w = (c.w & 0x7f7f7f7fu) + add4;
  return c;
}
__host__ __device__ __forceinline__ uint32_t dropout_thr7(float p) {
  int t = static_cast<int>(p * 128.f + 0.5f);
  return static_cast<uint32_t>(t < 0 ? 0 : (t > 127 ? 127 : t));
}
// byte permute with sign replication: selector nibble 8 + j spreads bit 7 of byte j
// over the whole destination byte
__device__ __forceinline__ uint32_t prmt_sign(uint32_t a, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(0u), "r"(selector));
  return d;
}
// keep word -> AND-mask for the 16-bit pair (2 k, 2 k + 1), k = 0 or 1
__device__ __forceinline__ uint32_t keep_mask_pair(uint32_t keep_word, int k) {
  return prmt_sign(keep_word, k == 0 ? 0x9988u : 0xBBAAu);
}
// keep word -> all-ones / zero 32-bit mask for element j (0..3)
__device__ __forceinline__ uint32_t keep_mask_full(uint32_t keep_word, int j) {
  return prmt_sign(keep_word, 0x8888u + 0x1111u * static_cast<uint32_t>(j));
}

// keep decisions for 8 consecutive elements starting at element index e0 (a
// multiple of 8): element e is byte (e % 16) of philox_keep16(index = e / 16),
// so the two threads that share a group of 16 elements evaluate the same call
// and each uses one half of its 16 draws.  The probability is quantised to
// thr7 / 128 like in the attention kernels; dropout_scale() is the matching
// 1 / (1 - p).
__device__ __forceinline__ void dropout_keep8(uint64_t seed, uint64_t offset, uint64_t e0,
                                              float p, bool keep[8]) {
  const uint32_t add4 = (128u - dropout_thr7(p)) * 0x01010101u;
  const uint4 c = philox_keep16(seed, offset, e0 >> 4, add4);
  const uint32_t lo = (e0 & 8) ? c.z : c.x, hi = (e0 & 8) ? c.w : c.y;
  keep[0] = lo & 0x80u; keep[1] = lo & 0x8000u; keep[2] = lo & 0x800000u; keep[3] = lo & 0x80000000u;
  keep[4] = hi & 0x80u; keep[5] = hi & 0x8000u; keep[6] = hi & 0x800000u; keep[7] = hi & 0x80000000u;
}
__host__ __device__ __forceinline__ float dropout_scale(float p) {
  return 128.f / (128.f - static_cast<float>(dropout_thr7(p)));
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

// erf by Abramowitz & Stegun 7.1.26 (|error| < 1.5e-7): one reciprocal, one exp2 and a
// degree-5 polynomial - about a third of the instructions of erff(), which matters because
// bias + GeLU on bf16 data has a budget of ~20 instructions per element before it becomes
// compute-bound on this GPU.  ``e`` returns exp(-x^2) for callers that need the Gaussian too.
__device__ __forceinline__ float erf_as(float x, float& e) {
  const float ax = fabsf(x);
  const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  e = exp2f(-1.4426950408889634f * ax * ax);
  return copysignf(fmaf(-poly * t, e, 1.f), x);
}

// activation codes shared with the Python side: 0 = GeLU (erf), 1 = GeLU (tanh), 2 = ReLU
__device__ __forceinline__ float act_fwd(float x, int act) {
  if (act == 0) {
    float e;
    return 0.5f * x * (1.f + erf_as(x * 0.70710678118654752f, e));
  }
  if (act == 1) {
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return fmaxf(x, 0.f);
}

__device__ __forceinline__ float act_grad(float x, int act) {
  if (act == 0) {
    float e;  // exp(-x^2 / 2): shared by the cdf's erf and the pdf
    const float cdf = 0.5f * (1.f + erf_as(x * 0.70710678118654752f, e));
    return fmaf(x * 0.3989422804014327f, e, cdf);
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
