// Flash attention forward on tcgen05 / TMEM (sm_100a).
//
// Tensors are [B, S, H, D] with D contiguous and arbitrary strides on B, S, H
// (so q/k/v slices of a fused QKV projection are read in place through 4-D
// TMA maps - no .contiguous() copies).  D is 64 or 128.
//
// One CTA handles 128 query rows of one (batch, head) and walks over the keys
// in tiles of 128:
//   warp 0    TMA: Q once, then a 2-deep K ring and a V buffer
//   warp 1    tcgen05.mma:  S = Q K^T  (fp32, 128 TMEM columns)
//                           O_j = P_j V_j  (fp32, double-buffered, D columns each)
//   warps 2-5 one query row per thread: read S from TMEM, online softmax in
//             the exp2 domain (scale, additive key bias, relative-position
//             bias, causal mask, Philox dropout), write P as bf16/fp16 into
//             swizzled shared memory for the second MMA, fold the per-tile O_j
//             into a register accumulator with the running rescale.
// The next S tile is issued before the previous P V product so the tensor
// core works while the softmax warps fold; for D = 64 two CTAs share an SM.
#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

#include <mutex>

namespace slapo {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_tmap_bshd(CUtensorMap* out, const void* base, uint64_t B, uint64_t S, uint64_t H,
                    uint64_t D, uint64_t stride_b, uint64_t stride_s, uint64_t stride_h,
                    uint32_t box_s, bool is_bf16) {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {D, H, S, B};
  cuuint64_t strides[3] = {stride_h * 2, stride_s * 2, stride_b * 2};
  cuuint32_t box[4] = {64, 1, box_s, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// ------------------------------------------------------------------------ //
constexpr int kBlockM = 128;   // query rows per CTA
constexpr int kBlockN = 128;   // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct FlashFwdParams {
  int B, H, Sq, Sk;
  int Dr;              // the tensors' head dimension (<= the kernel's tile width D, % 8 == 0):
                       // TMA zero-fills columns Dr .. D - 1 of every Q / K / V tile
  void* O;             // [B, Sq, H, Dr] contiguous
  float* lse;          // [B, H, Sq] natural-log sum-exp of the scaled scores
  const float* kbias;  // [B, Sk] additive key bias or nullptr
  const float* rel;    // [H, Sq + Sk - 1] additive bias by (key - query) + Sq - 1, or nullptr
  float scale_log2;    // softmax scale * log2(e)
  int causal;
  float p_drop;        // effective probability thr7 / 128
  uint32_t thr7;
  PhiloxArgs rng;
  int out_bf16;
  uint32_t idesc_qk, idesc_pv;
  int* status;
};

__device__ __forceinline__ uint32_t pack_pair(float a, float b, int bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// additive (log2-domain) score terms and masking for 32 consecutive keys
template <bool kFirstPass>
__device__ __forceinline__ void score_chunk(const uint32_t (&raw)[32], float (&v)[32], int row,
                                            int key0, const FlashFwdParams& p,
                                            const float* kb_tile, const float* rel_row,
                                            int key_limit, int col_in_tile) {
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int key = key0 + t;
    float s = __uint_as_float(raw[t]) * p.scale_log2;
    if (kb_tile != nullptr) s += kb_tile[col_in_tile + t];
    if (rel_row != nullptr) s += rel_row[key] * kLog2e;
    v[t] = key < key_limit ? s : -INFINITY;
  }
}

// kPlain: no key bias, no relative bias, not causal, Sk a multiple of 128 and a positive
// scale - the row maximum is then taken on the raw scores and every probability is one
// fused multiply-add plus one exp2.
template <int D, bool kPlain>
__global__ void __launch_bounds__(192, D == 64 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const FlashFwdParams p) {
  constexpr int kTileBytes = 128 * D * 2;   // one [128 x D] 16-bit tile
  constexpr int kBlkBytes = 128 * 128;      // one [128 rows x 64 cols] swizzled block
  constexpr int kDBlocks = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* s_q = smem;
  uint8_t* s_k = s_q + kTileBytes;          // 2 stages
  uint8_t* s_v = s_k + 2 * kTileBytes;
  uint8_t* s_p = s_v + kTileBytes;          // [128 x 128] 16-bit = 2 blocks
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + 2 * kBlkBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 6;
  uint64_t* s_full = bars + 7;
  uint64_t* p_full = bars + 8;
  uint64_t* o_full = bars + 9;        // 2
  uint64_t* o_empty = bars + 11;      // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* kb_tile = reinterpret_cast<float*>(bars + 16);  // 128 floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kBlockM;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int diag = p.Sk - p.Sq;  // key j visible to query i iff j <= i + diag (causal)
  int n_tiles = (p.Sk + kBlockN - 1) / kBlockN;
  if (p.causal) {
    const int last_key = min(p.Sk, q0 + kBlockM + diag);
    n_tiles = max(1, min(n_tiles, (last_key + kBlockN - 1) / kBlockN));
  }
  constexpr uint32_t kTmemCols = D == 64 ? 256 : 512;

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&k_full[i], 1);
      tc::mbar_init(&k_empty[i], 1);
      tc::mbar_init(&o_full[i], 1);
      tc::mbar_init(&o_empty[i], 4);
    }
    tc::mbar_init(v_full, 1);
    tc::mbar_init(v_empty, 1);
    tc::mbar_init(s_full, 1);
    tc::mbar_init(p_full, 4);
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
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tm_q);
      tc::tma_prefetch_desc(&tm_k);
      tc::tma_prefetch_desc(&tm_v);
      tc::mbar_arrive_expect_tx(q_full, kTileBytes);
#pragma unroll
      for (int d = 0; d < kDBlocks; ++d)
        tc::tma_load_4d(s_q + d * kBlkBytes, &tm_q, q_full, d * 64, head, q0, batch);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (!tc::mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc::mbar_arrive_expect_tx(&k_full[st], kTileBytes);
#pragma unroll
        for (int d = 0; d < kDBlocks; ++d)
          tc::tma_load_4d(s_k + st * kTileBytes + d * kBlkBytes, &tm_k, &k_full[st], d * 64, head,
                          j * kBlockN, batch);
        if (!tc::mbar_wait(v_empty, (j & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc::mbar_arrive_expect_tx(v_full, kTileBytes);
#pragma unroll
        for (int d = 0; d < kDBlocks; ++d)
          tc::tma_load_4d(s_v + d * kBlkBytes, &tm_v, v_full, d * 64, head, j * kBlockN, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = tc::mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_addr = tc::smem_u32(s_q);
      const uint32_t v_addr = tc::smem_u32(s_v);
      const uint32_t p_addr = tc::smem_u32(s_p);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        if (!tc::mbar_wait(&k_full[st], (j >> 1) & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t k_addr = tc::smem_u32(s_k + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBlkBytes + (kk & 3) * 32;
          tc::umma_f16(tmem_s, tc::smem_desc(q_addr + off, 16, 1024),
                       tc::smem_desc(k_addr + off, 16, 1024), p.idesc_qk, kk != 0 ? 1u : 0u);
        }
        tc::umma_commit(s_full);
        tc::umma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // P_j written (hence S_j fully read): S may be overwritten by the next tile
        if (!tc::mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        if (j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
        const int ob = j & 1;
        if (!tc::mbar_wait(&o_empty[ob], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        if (!tc::mbar_wait(v_full, j & 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          const uint64_t a_desc =
              tc::smem_desc(p_addr + (kk >> 2) * kBlkBytes + (kk & 3) * 32, 16, 1024);
          const uint64_t b_desc = tc::smem_desc(v_addr + kk * 2048, kBlkBytes, 1024);
          tc::umma_f16(tmem_o + ob * D, a_desc, b_desc, p.idesc_pv, kk != 0 ? 1u : 0u);
        }
        tc::umma_commit(&o_full[ob]);
        tc::umma_commit(v_empty);
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int row = q0 + row_in_tile;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int sm_tid = (warp - 2) * 32 + lane;
    uint64_t seed = 0, offset = 0;
    if (p.p_drop > 0.f) philox_unpack(p.rng, seed, offset);
    const uint32_t add4 = (128u - p.thr7) * 0x01010101u;
    const int sk16 = (p.Sk + 15) >> 4;
    const uint64_t drop_row_base =
        (static_cast<uint64_t>(batch * p.H + head) * p.Sq + min(row, p.Sq - 1)) * sk16;
    const float* rel_row = nullptr;
    if (p.rel != nullptr)
      rel_row = p.rel + static_cast<int64_t>(head) * (p.Sq + p.Sk - 1) + (p.Sq - 1) - min(row, p.Sq - 1);
    float o_acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o_acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_fold = 1.f;
    bool ok = true;

    auto fold = [&](int jt) -> bool {
      const int ob = jt & 1;
      if (!tc::mbar_wait_warp(&o_full[ob], (jt >> 1) & 1, abort_flag)) return false;
      tc::fence_after_sync();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_x32(tmem_o + ob * D + c * 32 + lane_sel, r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t)
          o_acc[c * 32 + t] = o_acc[c * 32 + t] * alpha_fold + __uint_as_float(r[t]);
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&o_empty[ob]);
      return true;
    };

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int k0 = j * kBlockN;
      if (p.kbias != nullptr) {
        softmax_bar_sync();  // previous tile's readers are done
        const int key = k0 + sm_tid;
        kb_tile[sm_tid] = key < p.Sk ? p.kbias[static_cast<int64_t>(batch) * p.Sk + key] * kLog2e : 0.f;
        softmax_bar_sync();
      }
      if (!tc::mbar_wait_warp(s_full, j & 1, abort_flag)) { ok = false; break; }
      tc::fence_after_sync();
      int key_limit = p.Sk;
      if (p.causal) key_limit = min(key_limit, row + diag + 1);
      const float* kb = p.kbias != nullptr ? kb_tile : nullptr;
      // pass 1: row maximum
      float mm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // 4 chains for ILP
#pragma unroll 1
      for (int c = 0; c < kBlockN / 32; ++c) {
        uint32_t raw[32];
        tc::tmem_ld_x32(tmem_s + c * 32 + lane_sel, raw);
        tc::tmem_ld_wait();
        if constexpr (kPlain) {
#pragma unroll
          for (int t = 0; t < 32; ++t) mm[t & 3] = fmaxf(mm[t & 3], __uint_as_float(raw[t]));
        } else {
          float v[32];
          score_chunk<true>(raw, v, row, k0 + c * 32, p, kb, rel_row, key_limit, c * 32);
#pragma unroll
          for (int t = 0; t < 32; ++t) mm[t & 3] = fmaxf(mm[t & 3], v[t]);
        }
      }
      float m_tile = fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3]));
      if constexpr (kPlain) m_tile *= p.scale_log2;
      const float m_new = fmaxf(m_run, m_tile);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m_run == -INFINITY ? 0.f : exp2f(m_run - m_use);
      // the P buffer is single: the previous P V product must have retired
      // before it is overwritten (the fold below consumes the same phase)
      if (j > 0 && !tc::mbar_wait_warp(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      // pass 2: probabilities, row sum, dropout, P -> shared memory
      float ll[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* p_row = s_p + row_in_tile * 128;
#pragma unroll 1
      for (int c = 0; c < kBlockN / 32; ++c) {
        uint32_t raw[32];
        float v[32];
        tc::tmem_ld_x32(tmem_s + c * 32 + lane_sel, raw);
        tc::tmem_ld_wait();
        if constexpr (kPlain) {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            v[t] = exp2f(fmaf(__uint_as_float(raw[t]), p.scale_log2, -m_use));
            ll[t & 3] += v[t];
          }
        } else {
          score_chunk<false>(raw, v, row, k0 + c * 32, p, kb, rel_row, key_limit, c * 32);
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            v[t] = exp2f(v[t] - m_use);
            ll[t & 3] += v[t];
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_pair(v[2 * i], v[2 * i + 1], p.out_bf16);
        if (p.p_drop > 0.f) {
          // dropped probabilities are cleared in the packed 16-bit pairs
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 kw = philox_keep16(seed, offset,
                                           drop_row_base + ((k0 + c * 32 + h * 16) >> 4), add4);
            const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              pk[h * 8 + i * 2 + 0] &= keep_mask_pair(w[i], 0);
              pk[h * 8 + i * 2 + 1] &= keep_mask_pair(w[i], 1);
            }
          }
        }
        // keys [c*32, c*32+32) of this row: block (c >> 1), 16-byte chunks (c & 1) * 4 + g
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;
          *reinterpret_cast<uint4*>(p_row + (c >> 1) * kBlkBytes +
                                    ((chunk ^ (row_in_tile & 7)) << 4)) =
              make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
        }
      }
      tc::fence_before_sync();   // S reads are complete
      tc::fence_proxy_async();   // P stores visible to the tensor core
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(p_full);
      l_run = l_run * alpha + ((ll[0] + ll[1]) + (ll[2] + ll[3]));
      if (j > 0) ok = fold(j - 1);
      alpha_fold = alpha;
      m_run = m_new;
    }
    if (ok) ok = fold(n_tiles - 1);
    if (ok && row < p.Sq) {
      const float inv = l_run > 0.f ? 1.f / (l_run * (1.f - p.p_drop)) : 0.f;
      uint8_t* dst = static_cast<uint8_t*>(p.O) +
                     ((static_cast<int64_t>(batch) * p.Sq + row) * p.H + head) * p.Dr * 2;
#pragma unroll
      for (int g = 0; g < D / 8; ++g) {
        if (g * 8 >= p.Dr) break;     // padded columns (zero) are not part of the output
        uint4 pk = make_uint4(pack_pair(o_acc[g * 8 + 0] * inv, o_acc[g * 8 + 1] * inv, p.out_bf16),
                              pack_pair(o_acc[g * 8 + 2] * inv, o_acc[g * 8 + 3] * inv, p.out_bf16),
                              pack_pair(o_acc[g * 8 + 4] * inv, o_acc[g * 8 + 5] * inv, p.out_bf16),
                              pack_pair(o_acc[g * 8 + 6] * inv, o_acc[g * 8 + 7] * inv, p.out_bf16));
        *reinterpret_cast<uint4*>(dst + g * 16) = pk;
      }
      const float m_nat = (m_run == -INFINITY ? 0.f : m_run) * 0.6931471805599453f;
      p.lse[(static_cast<int64_t>(batch) * p.H + head) * p.Sq + row] =
          l_run > 0.f ? m_nat + logf(l_run) : -INFINITY;
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 2);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Dropout keep-mask exactly as the attention kernels draw it (testing aid).
__global__ void flash_dropout_mask_kernel(uint8_t* mask, int B, int H, int Sq, int Sk, float p_drop,
                                          PhiloxArgs rng) {
  uint64_t seed, offset;
  philox_unpack(rng, seed, offset);
  const uint32_t add4 = (128u - dropout_thr7(p_drop)) * 0x01010101u;
  const int sk16 = (Sk + 15) >> 4;
  const int64_t total = static_cast<int64_t>(B) * H * Sq * sk16;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 kw = philox_keep16(seed, offset, static_cast<uint64_t>(i), add4);
    const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
    const int64_t rowi = i / sk16;
    const int k16 = static_cast<int>(i % sk16) * 16;
    for (int t = 0; t < 16; ++t)
      if (k16 + t < Sk) mask[rowi * Sk + k16 + t] = (w[t >> 2] >> (8 * (t & 3) + 7)) & 1u;
  }
}

void launch_flash_dropout_mask(uint8_t* mask, int B, int H, int Sq, int Sk, float p_drop,
                               PhiloxArgs rng, cudaStream_t stream) {
  count_launch();
  flash_dropout_mask_kernel<<<sm_count() * 4, 256, 0, stream>>>(mask, B, H, Sq, Sk, p_drop, rng);
}

template <int D, bool kPlain>
static int launch_fwd_d(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                        const FlashFwdParams& p, cudaStream_t stream) {
  constexpr int kSmem = 4 * 128 * D * 2 + 2 * 128 * 128 + 16 * 8 + 128 * 4 + 1024;
  auto kernel = flash_fwd_kernel<D, kPlain>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess)
      return 3;
    configured = true;
  }
  dim3 grid((p.Sq + kBlockM - 1) / kBlockM, p.H, p.B);
  count_launch();
  kernel<<<grid, 192, kSmem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int launch_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                     const float* kbias, const float* rel, int B, int H, int Sq, int Sk, int D,
                     const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                     float scale, int causal, float p_drop, PhiloxArgs rng, bool bf16, int* status,
                     cudaStream_t stream) {
  // any head dimension up to 128 that is a multiple of 8 (16-byte rows for TMA): the kernels
  // work on 64- or 128-wide tiles whose columns beyond D are zero-filled by the tile loads
  if (D < 8 || D > 128 || D % 8 != 0) return 1;
  const int Dt = D <= 64 ? 64 : 128;
  CUtensorMap tq, tk, tv;
  if (!make_tmap_bshd(&tq, q, B, Sq, H, D, q_strides[0], q_strides[1], q_strides[2], 128, bf16) ||
      !make_tmap_bshd(&tk, k, B, Sk, H, D, k_strides[0], k_strides[1], k_strides[2], 128, bf16) ||
      !make_tmap_bshd(&tv, v, B, Sk, H, D, v_strides[0], v_strides[1], v_strides[2], 128, bf16))
    return 2;
  FlashFwdParams p;
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.Dr = D; p.O = o; p.lse = lse; p.kbias = kbias; p.rel = rel;
  p.scale_log2 = scale * kLog2e; p.causal = causal; p.rng = rng;
  // the dropout probability is quantised to a multiple of 1/128 (see philox_keep16)
  p.thr7 = dropout_thr7(p_drop);
  p.p_drop = p.thr7 / 128.f;
  p.out_bf16 = bf16 ? 1 : 0; p.status = status;
  p.idesc_qk = tc::instr_desc_f16(128, 128, bf16 ? 1 : 0, false, false);
  p.idesc_pv = tc::instr_desc_f16(128, Dt, bf16 ? 1 : 0, false, true);
  const bool plain = kbias == nullptr && rel == nullptr && !causal && Sk % kBlockN == 0 && scale > 0.f;
  if (Dt == 64)
    return plain ? launch_fwd_d<64, true>(tq, tk, tv, p, stream)
                 : launch_fwd_d<64, false>(tq, tk, tv, p, stream);
  return plain ? launch_fwd_d<128, true>(tq, tk, tv, p, stream)
               : launch_fwd_d<128, false>(tq, tk, tv, p, stream);
}

}  // namespace slapo
