// CTA-pair tcgen05 GEMM for sm_100a: two CTAs of a cluster (one TPC) share every MMA.
//
//   C[M, N] = epilogue( A * B^T )        bf16 / fp16 inputs, fp32 accumulation
//
// Operand layouts as in gemm.cu (K-major or M/N-major A and B, so that forward, dgrad and
// wgrad of a linear layer need no transposes).  A pair works on a 256 x BN output tile:
// `tcgen05.mma.cta_group::2` with M = 256, N = BN, K = 16, issued by one thread of the pair's
// leader CTA.  Each CTA loads ITS 128 rows of A and ITS BN / 2 rows of B (plain tile loads into
// its own shared memory) and ends up with ITS 128 x BN fp32 accumulator rows in its tensor
// memory - per SM half the B traffic of a 128 x BN single-CTA tile, which is what lifts the
// shared-memory and L2 ceilings of the single-CTA kernel.
//
// Hand-offs (all mbarriers, all waits bounded):
//   full[s]    in the leader; both producers arrive with their own byte count, all loads of
//              the pair complete their bytes on it
//   empty[s]   in each CTA; the leader's MMA thread commits to both after the MMAs of a stage
//   tmem_full[a]   in each CTA; committed to both when a tile's accumulator is complete
//   tmem_empty[a]  in the leader; the eight epilogue warps of the pair arrive on it
//
// Split-K (few output tiles, long contraction - weight gradients): `splits` CTA pairs share
// a tile, each stores its partial accumulator into its own fp32 slice of a workspace; a
// second, memory-bound kernel adds the slices, applies bias / activation and writes C.
#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace slapo {

struct Gemm2Params {
  int M, N, K;
  void* C;
  void* C2;           // optional second output: the value before the activation
  int ldc;
  const void* bias;   // [N] or nullptr
  int act;            // -1 none
  int out_bf16;
  uint32_t idesc;
  int splits;         // CTA pairs per output tile (>= 1)
  int kb_per_split;
  float* workspace;   // [splits, M, N] fp32 scratch (splits > 1), any contents
  int* status;
  int wide_store;     // rows of C are 32-byte aligned: the epilogue stores whole sectors
};

constexpr int kEpiWarps = 8;   // epilogue warps per CTA: two per quarter of the tensor-memory lanes,
                               // each taking half of the tile's columns
constexpr int PBM = 128;   // rows of A per CTA (the pair's tile has 256)
constexpr int PBK = 64;
#ifndef SLAPO_GEMM2_KSUB
#define SLAPO_GEMM2_KSUB 2
#endif
constexpr int kKSub = SLAPO_GEMM2_KSUB;   // k-blocks of 64 per pipeline stage

// A pipeline stage holds KSUB k-blocks of 64 (each its own 128-byte-swizzled sub-tile): with
// KSUB = 2 the producer / MMA hand-off (barrier wait, two commits) happens once per 128 of K
// instead of once per 64.
template <int BN, int STAGES, int KSUB>
struct Gemm2Smem {
  static constexpr int kASub = PBM * PBK * 2;
  static constexpr int kBSub = (BN / 2) * PBK * 2;
  static constexpr int kABytes = KSUB * kASub;
  static constexpr int kBBytes = KSUB * kBSub;
  static constexpr int kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

__device__ __forceinline__ uint32_t g2_pack2(float a, float b, int out_bf16) {
  if (out_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float g2_bias(const void* bias, int col, int out_bf16) {
  if (out_bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[col]);
  return __half2float(static_cast<const __half*>(bias)[col]);
}

// bias + activation + pack + store of 32 consecutive columns of one row.  (Staging the tile in
// shared memory for whole-line or TMA stores was measured and lost by a factor of two: the
// epilogue's shared-memory traffic then competes with the operand fetch of the MMAs that run
// under it.  Direct stores of whole 32-byte sectors are what is kept.)
// the 32 bias values of columns [col0, col0 + 32): four 16-byte loads (the same for every
// row, so they hit L1) instead of one 2-byte load per element; zeros without a bias
__device__ __forceinline__ void g2_load_bias(const Gemm2Params& p, int col0, uint32_t (&b)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 t = make_uint4(0u, 0u, 0u, 0u);
    if (p.bias != nullptr && col0 + q * 8 < p.N)
      t = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.bias) +
                                               (col0 + q * 8) * 2));
    b[4 * q] = t.x; b[4 * q + 1] = t.y; b[4 * q + 2] = t.z; b[4 * q + 3] = t.w;
  }
}

__device__ __forceinline__ void g2_finish_store(const Gemm2Params& p, const float (&v)[32], int row,
                                                int col0, const uint32_t (&bias_raw)[16]) {
  uint32_t packed[16], packed2[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float v0 = v[2 * j], v1 = v[2 * j + 1];
    if (p.bias != nullptr) {
      float2 b2;
      if (p.out_bf16) b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bias_raw[j]));
      else b2 = __half22float2(*reinterpret_cast<const __half2*>(&bias_raw[j]));
      v0 += b2.x;
      v1 += b2.y;
    }
    if (p.C2 != nullptr) packed2[j] = g2_pack2(v0, v1, p.out_bf16);
    if (p.act >= 0) {
      v0 = act_fwd(v0, p.act);
      v1 = act_fwd(v1, p.act);
    }
    packed[j] = g2_pack2(v0, v1, p.out_bf16);
  }
  const int64_t off = (static_cast<int64_t>(row) * p.ldc + col0) * 2;
  uint8_t* dst = static_cast<uint8_t*>(p.C) + off;
  if (p.wide_store) {
    // whole 32-byte sectors per store (rows are 32-byte aligned: checked by the launcher)
#pragma unroll
    for (int q = 0; q < 2; ++q)
      if (col0 + q * 16 + 8 < p.N)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + q * 32),
                     "r"(packed[8 * q]), "r"(packed[8 * q + 1]), "r"(packed[8 * q + 2]),
                     "r"(packed[8 * q + 3]), "r"(packed[8 * q + 4]), "r"(packed[8 * q + 5]),
                     "r"(packed[8 * q + 6]), "r"(packed[8 * q + 7])
                     : "memory");
      else if (col0 + q * 16 < p.N)
        *reinterpret_cast<uint4*>(dst + q * 32) = make_uint4(
            packed[8 * q], packed[8 * q + 1], packed[8 * q + 2], packed[8 * q + 3]);
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (col0 + q * 8 < p.N)
        *reinterpret_cast<uint4*>(dst + q * 16) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
  }
  if (p.C2 != nullptr) {
    uint8_t* dst2 = static_cast<uint8_t*>(p.C2) + off;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (col0 + q * 8 < p.N)
        *reinterpret_cast<uint4*>(dst2 + q * 16) =
            make_uint4(packed2[4 * q], packed2[4 * q + 1], packed2[4 * q + 2], packed2[4 * q + 3]);
  }
}

template <int BN, int STAGES, int KSUB, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * kEpiWarps, 1)
gemm2_tc05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const Gemm2Params p) {
  using S = Gemm2Smem<BN, STAGES, KSUB>;
  constexpr int HBN = BN / 2;   // rows of B per CTA
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
  const uint32_t cta = tc::cluster_ctarank();        // 0 = leader of the pair
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int npairs = static_cast<int>(gridDim.x >> 1);
  const int tiles_m = (p.M + 2 * PBM - 1) / (2 * PBM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + PBK - 1) / PBK;
  const int units = tiles_m * tiles_n * p.splits;
  constexpr uint32_t kTmemCols = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_bar[s], 2);    // one arrival (with its byte count) per producer
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&tmem_full[a], 1);
      tc::mbar_init(&tmem_empty[a], 2 * kEpiWarps);  // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc_pair(tmem_slot, kTmemCols);
    tc::tmem_relinquish_pair();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::cluster_sync_all();   // the peer's barriers are initialised before anything targets them
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmap_a);
      tc::tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += npairs) {
        const int tile = u / p.splits, sp = u - tile * p.splits;
        const int m0 = (tile / tiles_n) * (2 * PBM) + static_cast<int>(cta) * PBM;
        const int n0 = (tile % tiles_n) * BN + static_cast<int>(cta) * HBN;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; kb += KSUB) {
          if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t bar = tc::map_to_cta(tc::smem_u32(&full_bar[stage]), 0);
          tc::mbar_arrive_expect_tx_cluster(bar, S::kABytes + S::kBBytes);
#pragma unroll
          for (int s = 0; s < KSUB; ++s) {
            // a k-block beyond K (last stage of an odd count) is zero-filled by the tile load
            const int kc = (kb + s) * PBK;
            const uint32_t sa = tc::smem_u32(smem_a + stage * S::kABytes + s * S::kASub);
            const uint32_t sb = tc::smem_u32(smem_b + stage * S::kBBytes + s * S::kBSub);
            if constexpr (!A_MN) {
              tc::tma_load_2d_pair(sa, &tmap_a, bar, kc, m0);
            } else {
#pragma unroll
              for (int j = 0; j < PBM / 64; ++j)
                tc::tma_load_2d_pair(sa + j * (PBK * 128), &tmap_a, bar, m0 + j * 64, kc);
            }
            if constexpr (!B_MN) {
              tc::tma_load_2d_pair(sb, &tmap_b, bar, kc, n0);
            } else {
#pragma unroll
              for (int j = 0; j < HBN / 64; ++j)
                tc::tma_load_2d_pair(sb + j * (PBK * 128), &tmap_b, bar, n0 + j * 64, kc);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) -----------------------------
    if (lane == 0 && cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += npairs, ++iter) {
        const int tile = u / p.splits, sp = u - tile * p.splits;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(num_kb, kb0 + p.kb_per_split);
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!tc::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb += KSUB) {
          if (!tc::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc::fence_after_sync();
#pragma unroll
          for (int s = 0; s < KSUB; ++s) {
            const uint32_t a_addr = tc::smem_u32(smem_a + stage * S::kABytes + s * S::kASub);
            const uint32_t b_addr = tc::smem_u32(smem_b + stage * S::kBBytes + s * S::kBSub);
#pragma unroll
            for (int k = 0; k < PBK / 16; ++k) {
              const uint64_t a_desc = A_MN ? tc::smem_desc(a_addr + k * 2048, PBK * 128, 1024)
                                           : tc::smem_desc(a_addr + k * 32, 16, 1024);
              const uint64_t b_desc = B_MN ? tc::smem_desc(b_addr + k * 2048, PBK * 128, 1024)
                                           : tc::smem_desc(b_addr + k * 32, 16, 1024);
              tc::umma_f16_pair(d_tmem, a_desc, b_desc, p.idesc,
                                (kb > kb0 || s != 0 || k != 0) ? 1u : 0u);
            }
          }
          // the stage is reusable in both CTAs once these MMAs retire
          const uint32_t eb = tc::smem_u32(&empty_bar[stage]);
          tc::umma_commit_pair(tc::map_to_cta(eb, 0));
          tc::umma_commit_pair(tc::map_to_cta(eb, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t fb = tc::smem_u32(&tmem_full[acc]);
          tc::umma_commit_pair(tc::map_to_cta(fb, 0));
          tc::umma_commit_pair(tc::map_to_cta(fb, 1));
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    // with eight warps, warps w and w + 4 share a quarter and split the columns
    const int col_part = (warp - 2) >> 2, col_parts = kEpiWarps / 4;
    constexpr int kChunks = BN / 32;
    const int c_begin = col_part * (kChunks / col_parts), c_end = c_begin + kChunks / col_parts;
    int iter = 0;
    bool ok = true;
    for (int u = pair; u < units && ok; u += npairs, ++iter) {
      const int tile = u / p.splits;
      const int m0 = (tile / tiles_n) * (2 * PBM) + static_cast<int>(cta) * PBM;
      const int n0 = (tile % tiles_n) * BN;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!tc::mbar_wait_warp(&tmem_full[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc::fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (p.splits == 1) {
        // One tensor-memory load at a time on purpose: reading ahead (two register sets, or
        // 64 columns per load) measured 20 - 30 % slower on whole GEMMs - the epilogue's
        // reads compete with the accumulator traffic of the MMAs that run under it.  Only the
        // bias words are fetched one chunk ahead.
        uint32_t bias_cur[16], bias_next[16];
        g2_load_bias(p, n0 + c_begin * 32, bias_next);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
#pragma unroll
          for (int j = 0; j < 16; ++j) bias_cur[j] = bias_next[j];
          if (c + 1 < c_end) g2_load_bias(p, n0 + (c + 1) * 32, bias_next);
          uint32_t r[32];
          tc::tmem_ld_x32(t_row + c * 32, r);
          tc::tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            g2_finish_store(p, v, row, col0, bias_cur);
          }
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_cta(tc::smem_u32(&tmem_empty[acc]), 0));
      } else {
        // this split's partial tile goes into ITS slice of the fp32 workspace with plain
        // stores; splitk_reduce_kernel adds the slices up afterwards with the whole GPU.
        // (fp32 atomics on rows 4 KB apart measured 0.8 TB/s, and a "last CTA to arrive sums
        // the slices" epilogue 70 us of serial loads: both slower than not splitting)
        const int sp = u - tile * p.splits;
        const int64_t slice = static_cast<int64_t>(p.M) * p.N;
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          tc::tmem_ld_x32(t_row + c * 32, r);
          tc::tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) {
            float* w = p.workspace + sp * slice + static_cast<int64_t>(row) * p.N + col0;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (col0 + q * 4 < p.N)
                __stcg(reinterpret_cast<float4*>(w + q * 4),
                       make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                   __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
          }
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_cta(tc::smem_u32(&tmem_empty[acc]), 0));
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
  // neither CTA may leave while the other can still signal its barriers or use its tensor memory
  tc::cluster_sync_all();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// C = act(sum of the split-K slices + bias): one thread per 8 columns, 16-byte stores
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const Gemm2Params p) {
  const int vpr = p.N / 8;
  const int64_t n_vec = static_cast<int64_t>(p.M) * vpr;
  const int64_t slice = static_cast<int64_t>(p.M) * p.N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / vpr);
    const int col = static_cast<int>(i - static_cast<int64_t>(row) * vpr) * 8;
    const float* w = p.workspace + static_cast<int64_t>(row) * p.N + col;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s2 = 0; s2 < p.splits; ++s2) {
      const float4 t0 = __ldcs(reinterpret_cast<const float4*>(w + s2 * slice));
      const float4 t1 = __ldcs(reinterpret_cast<const float4*>(w + s2 * slice + 4));
      v[0] += t0.x; v[1] += t0.y; v[2] += t0.z; v[3] += t0.w;
      v[4] += t1.x; v[5] += t1.y; v[6] += t1.z; v[7] += t1.w;
    }
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v0 = v[2 * j], v1 = v[2 * j + 1];
      if (p.bias != nullptr) {
        v0 += g2_bias(p.bias, col + 2 * j, p.out_bf16);
        v1 += g2_bias(p.bias, col + 2 * j + 1, p.out_bf16);
      }
      if (p.act >= 0) {
        v0 = act_fwd(v0, p.act);
        v1 = act_fwd(v1, p.act);
      }
      packed[j] = g2_pack2(v0, v1, p.out_bf16);
    }
    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.C) +
                              (static_cast<int64_t>(row) * p.ldc + col) * 2) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// ------------------------------------------------------------------------ //
bool cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                    uint64_t stride, uint32_t box_outer, bool bf16);

template <int BN, int STAGES, int KSUB, bool A_MN, bool B_MN>
static int launch_pair_variant(const CUtensorMap& ta, const CUtensorMap& tb, const Gemm2Params& p,
                               cudaStream_t stream) {
  using S = Gemm2Smem<BN, STAGES, KSUB>;
  auto kernel = gemm2_tc05_kernel<BN, STAGES, KSUB, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) !=
        cudaSuccess)
      return 3;
    configured = true;
  }
  const int units = ((p.M + 2 * PBM - 1) / (2 * PBM)) * ((p.N + BN - 1) / BN) * p.splits;
  const int pairs = sm_count() / 2;
  const int grid = 2 * (units < pairs ? units : pairs);
  count_launch();
  kernel<<<grid, 64 + 32 * kEpiWarps, S::kTotal, stream>>>(ta, tb, p);
  if (p.splits > 1) {
    const int64_t n_vec = static_cast<int64_t>(p.M) * (p.N / 8);
    const int64_t blocks = (n_vec + 255) / 256;
    const int cap = sm_count() * 8;
    count_launch();
    splitk_reduce_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// Number of CTA pairs that share one output tile: 1 unless the tiles alone leave most of the
// GPU idle and the contraction is long enough to be cut (at least 8 k-blocks per pair).
int gemm2_splits(int M, int N, int K, int bn) {
  const int tiles = ((M + 2 * PBM - 1) / (2 * PBM)) * ((N + bn - 1) / bn);
  const int pairs = sm_count() / 2;
  const int num_kb = (K + PBK - 1) / PBK;
  if (tiles * 2 > pairs || num_kb < 16) return 1;
  int s = pairs / tiles;
  if (s > 16) s = 16;
  if (s > num_kb / 8) s = num_kb / 8;
  if (s < 1) s = 1;
  const int per = (num_kb + s - 1) / s;
  return (num_kb + per - 1) / per;     // no empty split
}

// C = act(A B^T + bias) on CTA pairs.  `workspace`: scratch for split-K, gemm2_splits() * M * N
// floats of any contents, or null (no split).
// Returns 0 on success; >0 = refused on the host (shape / alignment / driver), 5 = too small
// for a pair tile (use launch_gemm).
int launch_gemm2(const void* A, const void* B, void* C, void* C2, const void* bias, int M, int N,
                 int K, int lda, int ldb, int ldc, bool a_mn, bool b_mn, bool bf16, int act,
                 float* workspace, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 8 || K % 8 || lda % 8 || ldb % 8 || ldc % 8) return 1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(C2)) & 15)
    return 1;
  if (a_mn && M % 8) return 1;
  if (M <= PBM || N <= 64) return 5;
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap ta, tb;
  bool ok = a_mn ? cached_tmap_2d(&ta, A, M, K, lda, PBK, bf16)
                 : cached_tmap_2d(&ta, A, K, M, lda, PBM, bf16);
  if (!ok) return 2;
  ok = b_mn ? cached_tmap_2d(&tb, B, N, K, ldb, PBK, bf16)
            : cached_tmap_2d(&tb, B, K, N, ldb, BN / 2, bf16);
  if (!ok) return 2;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.C2 = C2; p.ldc = ldc; p.bias = bias; p.act = act;
  p.out_bf16 = bf16 ? 1 : 0; p.status = status;
  p.wide_store = (ldc % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 31) == 0) ? 1 : 0;
  p.idesc = tc::instr_desc_f16(2 * PBM, BN, bf16 ? 1 : 0, a_mn, b_mn);
  p.splits = workspace != nullptr ? gemm2_splits(M, N, K, BN) : 1;

  const int num_kb = (K + PBK - 1) / PBK;
  p.kb_per_split = (num_kb + p.splits - 1) / p.splits;
  p.kb_per_split = (p.kb_per_split + kKSub - 1) / kKSub * kKSub;   // whole pipeline stages
  p.splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.workspace = workspace;

#define GEMM2_CASE(BN_, ST_)                                                                  \
  if (BN == BN_) {                                                                            \
    if (!a_mn && !b_mn)                                                                       \
      return launch_pair_variant<BN_, ST_, kKSub, false, false>(ta, tb, p, stream);            \
    if (!a_mn && b_mn) return launch_pair_variant<BN_, ST_, kKSub, false, true>(ta, tb, p, stream); \
    if (a_mn && !b_mn) return launch_pair_variant<BN_, ST_, kKSub, true, false>(ta, tb, p, stream); \
    return launch_pair_variant<BN_, ST_, kKSub, true, true>(ta, tb, p, stream);                \
  }
  GEMM2_CASE(256, 6 / kKSub)
  GEMM2_CASE(128, 8 / kKSub)
#undef GEMM2_CASE
  return 1;
}

}  // namespace slapo
