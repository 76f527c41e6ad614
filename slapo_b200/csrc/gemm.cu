// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M, N] = epilogue( A * B^T )        bf16 / fp16 inputs, fp32 accumulation
//
//   A: K-major  [M, K] (row-major, K contiguous)   or M-major [K, M]
//   B: K-major  [N, K] (row-major, K contiguous)   or N-major [K, N]
//
// so the three GEMMs of a linear layer are all covered without transposes:
//   forward  Y  = X  W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad    dX = dY W        A = dY (K-major)   B = W  (N-major: [N_w, K_w] read as [K, N])
//   wgrad    dW = dY^T X      A = dY (M-major)   B = X  (N-major)
//
// One CTA per SM loops over 128 x BN output tiles.  Warp 0 feeds a STAGES-deep
// shared-memory ring with TMA tile loads (128-byte swizzle), warp 1 issues
// tcgen05.mma (M = 128, N = BN, K = 16) into one of two TMEM accumulators,
// warps 2-5 drain the other accumulator with tcgen05.ld, apply the epilogue
// (bias, activation) and store 16-byte vectors.  All hand-offs are mbarriers;
// every wait is bounded and reports through a device status word.
#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

#include <mutex>
#include <unordered_map>

namespace slapo {

// ------------------------------------------------------------------------ //
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                  uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer,
                  int elem_bytes, bool is_bf16) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// ------------------------------------------------------------------------ //
struct GemmParams {
  int M, N, K;
  void* C;
  int ldc;
  const void* bias;   // [N] or nullptr
  int act;            // -1 none, else activation code applied after the bias
  int out_bf16;       // 1 bf16, 0 fp16
  uint32_t idesc;
  int* status;        // device error word (0 = ok)
};

constexpr int BM = 128;
constexpr int BK = 64;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // + barriers + alignment slack
};

__device__ __forceinline__ uint32_t pack2(float a, float b, int out_bf16) {
  if (out_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float load_bias(const void* bias, int col, int out_bf16) {
  if (out_bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[col]);
  return __half2float(static_cast<const __half*>(bias)[col]);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * S::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&tmem_full[a], 1);
      tc::mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmap_a);
      tc::tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * BM;
        const int n0 = (tile % tiles_n) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(&full_bar[stage], S::kABytes + S::kBBytes);
          uint8_t* sa = smem_a + stage * S::kABytes;
          uint8_t* sb = smem_b + stage * S::kBBytes;
          if constexpr (!A_MN) {
            tc::tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tc::tma_load_2d(sa + j * (BK * 128), &tmap_a, &full_bar[stage], m0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tc::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tc::tma_load_2d(sb + j * (BK * 128), &tmap_b, &full_bar[stage], n0 + j * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!tc::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc::fence_after_sync();
          const uint32_t a_addr = tc::smem_u32(smem_a + stage * S::kABytes);
          const uint32_t b_addr = tc::smem_u32(smem_b + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t a_desc = A_MN ? tc::smem_desc(a_addr + k * 2048, BK * 128, 1024)
                                         : tc::smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = B_MN ? tc::smem_desc(b_addr + k * 2048, BK * 128, 1024)
                                         : tc::smem_desc(b_addr + k * 32, 16, 1024);
            tc::umma_f16(d_tmem, a_desc, b_desc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc::umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc::umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
      const int m0 = (tile / tiles_n) * BM;
      const int n0 = (tile % tiles_n) * BN;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!tc::mbar_wait_warp(&tmem_full[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc::fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_x32(t_row + c * 32, r);
        tc::tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v0 = __uint_as_float(r[2 * j]);
            float v1 = __uint_as_float(r[2 * j + 1]);
            if (p.bias != nullptr) {
              const int cc = min(col0 + 2 * j, p.N - 2);
              v0 += load_bias(p.bias, cc, p.out_bf16);
              v1 += load_bias(p.bias, cc + 1, p.out_bf16);
            }
            if (p.act >= 0) {
              v0 = act_fwd(v0, p.act);
              v1 = act_fwd(v1, p.act);
            }
            packed[j] = pack2(v0, v1, p.out_bf16);
          }
          uint8_t* dst = static_cast<uint8_t*>(p.C) +
                         (static_cast<int64_t>(row) * p.ldc + col0) * 2;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N)
              *reinterpret_cast<uint4*>(dst + v * 16) =
                  make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------ //
struct TmapKey {
  const void* base; uint64_t inner, outer, stride; uint32_t box_outer; int bf16;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride &&
           box_outer == o.box_outer && bf16 == o.bf16;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.inner; h = h * 1000003u ^ k.outer; h = h * 1000003u ^ k.stride;
    h = h * 1000003u ^ k.box_outer; h = h * 1000003u ^ static_cast<size_t>(k.bf16);
    return h;
  }
};

bool cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                    uint64_t stride, uint32_t box_outer, bool bf16) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{base, inner, outer, stride, box_outer, bf16 ? 1 : 0};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  if (!make_tmap_2d(out, base, inner, outer, stride, 64, box_outer, 2, bf16)) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                          cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kernel = gemm_tc05_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) !=
        cudaSuccess)
      return 3;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  count_launch();
  kernel<<<grid, 192, S::kTotal, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// Returns 0 on success; >0 = host-side refusal (bad shape / alignment / driver).
int launch_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                int lda, int ldb, int ldc, bool a_mn, bool b_mn, bool bf16, int act, int* status,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 8 || K % 8 || lda % 8 || ldb % 8 || ldc % 8) return 1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return 1;
  if (a_mn && M % 8) return 1;
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap ta, tb;
  bool ok;
  // K-major: [rows, K] -> inner K, outer rows, box 64 x rows_per_tile
  // MN-major: [K, rows] -> inner rows, outer K, box 64 x BK
  ok = a_mn ? cached_tmap_2d(&ta, A, M, K, lda, BK, bf16) : cached_tmap_2d(&ta, A, K, M, lda, BM, bf16);
  if (!ok) return 2;
  ok = b_mn ? cached_tmap_2d(&tb, B, N, K, ldb, BK, bf16) : cached_tmap_2d(&tb, B, K, N, ldb, BN, bf16);
  if (!ok) return 2;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.bias = bias; p.act = act;
  p.out_bf16 = bf16 ? 1 : 0; p.status = status;
  p.idesc = tc::instr_desc_f16(BM, BN, bf16 ? 1 : 0, a_mn, b_mn);

#define GEMM_CASE(BN_, ST_)                                                              \
  if (BN == BN_) {                                                                       \
    if (!a_mn && !b_mn) return launch_variant<BN_, ST_, false, false>(ta, tb, p, stream); \
    if (!a_mn && b_mn) return launch_variant<BN_, ST_, false, true>(ta, tb, p, stream);   \
    if (a_mn && !b_mn) return launch_variant<BN_, ST_, true, false>(ta, tb, p, stream);   \
    return launch_variant<BN_, ST_, true, true>(ta, tb, p, stream);                       \
  }
  GEMM_CASE(256, 4)
  GEMM_CASE(128, 6)
  GEMM_CASE(64, 8)
#undef GEMM_CASE
  return 1;
}

}  // namespace slapo
