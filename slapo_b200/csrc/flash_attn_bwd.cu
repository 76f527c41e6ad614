// Flash attention backward on tcgen05 / TMEM (sm_100a).
//
// One CTA owns 128 keys of one (batch, head) and walks over the query tiles
// (128 rows) that can see them.  Per query tile:
//   tensor core   S  = Q K^T            dP = dO V^T                (fp32 in TMEM)
//   128 threads   p  = exp2(s - lse),   ds = p * (dp - delta)      (one query row each,
//                 Philox dropout replayed), P and scale*dS written as 16-bit
//                 tiles into swizzled shared memory
//   tensor core   dV += P^T dO          dK += dS^T Q               (TMEM accumulators
//                 dQ_tile = dS K                                    over all query tiles)
//   128 threads   dQ_tile -> fp32 partial of this key tile (plain 16-byte stores; the
//                 conversion kernel sums the partials), or, for very long key sequences,
//                 a shared fp32 accumulator (vector red.add)
// The same shared-memory bytes serve as K-major and M/N-major operands: only
// the descriptors differ, nothing is transposed.  delta = rowsum(dO * O) comes
// from a small pre-pass; the fp32 dQ accumulator is converted by the caller.
#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace slapo {

constexpr float kLog2eB = 1.4426950408889634f;

struct FlashBwdParams {
  int B, H, Sq, Sk;
  int Dr;               // the tensors' head dimension (<= the tile width D, % 8 == 0)
  const float* lse;     // [B, H, Sq]
  const float* delta;   // [B, H, Sq]
  float* dq_accum;      // [B, Sq, H, Dr] fp32, zero-initialised (dq_slice_stride == 0), or one
                        // such partial per 128-key tile, written with plain stores
  int64_t dq_slice_stride;
  void* dK;             // rows (b, key, head) spaced dkv_row_stride elements apart
  void* dV;
  int64_t dkv_row_stride;  // D for contiguous [B, Sk, H, D]; 3 D inside a packed QKV gradient
  const float* kbias;   // [B, Sk] or nullptr
  const float* rel;     // [H, Sq + Sk - 1] or nullptr
  float* drel;          // same shape fp32 accumulator or nullptr
  float scale, scale_log2;
  int causal;
  float p_drop;         // effective probability thr7 / 128
  uint32_t thr7;
  PhiloxArgs rng;
  int bf16;
  uint32_t idesc_s, idesc_dvk, idesc_dq;
  int* status;
};

__device__ __forceinline__ uint32_t pack_pair_b(float a, float b, int bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]   (both contiguous [B, Sq, H, Dr]).
// D / 8 lanes share a row (16-byte loads), D = Dr rounded up to 64 or 128, so a warp covers
// 256 / D rows; lanes beyond Dr / 8 contribute zero.
template <typename T>
__global__ void flash_bwd_delta_kernel(const T* __restrict__ dout, const T* __restrict__ out,
                                       float* __restrict__ delta, int B, int H, int Sq, int D,
                                       int Dr) {
  const int lanes_per_row = D >> 3;              // 8 (D = 64) or 16 (D = 128)
  const int rows_per_warp = 32 / lanes_per_row;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const int64_t row = warp_id * rows_per_warp + lane / lanes_per_row;
  const int64_t rows = static_cast<int64_t>(B) * Sq * H;
  float s = 0.f;
  const int d = (lane % lanes_per_row) * 8;
  if (row < rows && d < Dr) {
    float a[8], b[8];
    Vec8<T>::load(dout + row * Dr + d, a);
    Vec8<T>::load(out + row * Dr + d, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += a[k] * b[k];
  }
  for (int o = lanes_per_row >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (row < rows && lane % lanes_per_row == 0) {
    const int h = static_cast<int>(row % H);
    const int64_t bi = row / H;
    const int i = static_cast<int>(bi % Sq);
    const int b = static_cast<int>(bi / Sq);
    delta[(static_cast<int64_t>(b) * H + h) * Sq + i] = s;
  }
}

// 10 warps: TMA, MMA and 8 softmax warps.  Softmax warps w and w + 4 share a quarter of the
// TMEM lanes (query rows) and split the 128 key columns (and later the D output columns)
// in halves, so every scheduler of the SM has two of them to interleave.
// kPlain: no key bias / relative bias, not causal, Sq and Sk multiples of 128.
template <int D, bool kPlain>
__global__ void __launch_bounds__(320, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const FlashBwdParams p) {
  constexpr int kTileBytes = 128 * D * 2;
  constexpr int kBlkBytes = 128 * 128;
  constexpr int kDBlocks = D / 64;
  constexpr int kStages = D == 64 ? 2 : 1;
  // D = 64: two P / dS buffers, so that the softmax warps write the tiles of query block j + 1
  // while the tensor core still reads those of block j (dV, dK, dQ); D = 128 has no room
  constexpr int kPB = D == 64 ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* s_k = smem;
  uint8_t* s_v = s_k + kTileBytes;
  uint8_t* s_q = s_v + kTileBytes;                  // kStages
  uint8_t* s_do = s_q + kStages * kTileBytes;       // kStages
  uint8_t* s_p = s_do + kStages * kTileBytes;       // kPB buffers of [P: 2 blocks | dS: 2 blocks]
  uint8_t* s_ds = s_p + 2 * kBlkBytes;
  constexpr int kPdsBytes = 4 * kBlkBytes;          // distance between the P / dS buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + kPB * kPdsBytes);
  uint64_t* kv_full = bars;            // 1
  uint64_t* qdo_full = bars + 1;       // kStages (<= 2)
  uint64_t* qdo_empty = bars + 3;      // kStages
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_full = bars + 6;       // 4 arrivals
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_empty = bars + 8;       // 4 arrivals
  uint64_t* acc_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* kb_tile = reinterpret_cast<float*>(bars + 12);  // 128 floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int diag = p.Sk - p.Sq;
  const int q_tiles = (p.Sq + 127) / 128;
  int i_begin = 0;
  if (p.causal) i_begin = max(0, (n0 - diag) / 128);
  i_begin = min(i_begin, q_tiles);
  const int n_iter = q_tiles - i_begin;

  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 256 + D;
  constexpr uint32_t kColDQ = D == 64 ? 384 : 0;  // D = 128: dQ reuses the S columns

  if (threadIdx.x == 0) {
    tc::mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(&qdo_full[s], 1);
      tc::mbar_init(&qdo_empty[s], 1);
    }
    tc::mbar_init(sdp_full, 1);
    tc::mbar_init(pds_full, 8);
    tc::mbar_init(dq_full, 1);
    tc::mbar_init(dq_empty, 8);
    tc::mbar_init(acc_full, 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  if (warp >= 2 && warp < 6) {
    const int t = (warp - 2) * 32 + lane;
    const int key = n0 + t;
    kb_tile[t] = (p.kbias != nullptr && key < p.Sk)
                     ? p.kbias[static_cast<int64_t>(batch) * p.Sk + key] * kLog2eB : 0.f;
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tm_q);
      tc::tma_prefetch_desc(&tm_do);
      tc::mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
#pragma unroll
      for (int d = 0; d < kDBlocks; ++d) {
        tc::tma_load_4d(s_k + d * kBlkBytes, &tm_k, kv_full, d * 64, head, n0, batch);
        tc::tma_load_4d(s_v + d * kBlkBytes, &tm_v, kv_full, d * 64, head, n0, batch);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!tc::mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        tc::mbar_arrive_expect_tx(&qdo_full[st], 2 * kTileBytes);
        const int m0 = (i_begin + it) * 128;
#pragma unroll
        for (int d = 0; d < kDBlocks; ++d) {
          tc::tma_load_4d(s_q + st * kTileBytes + d * kBlkBytes, &tm_q, &qdo_full[st], d * 64, head,
                          m0, batch);
          tc::tma_load_4d(s_do + st * kTileBytes + d * kBlkBytes, &tm_do, &qdo_full[st], d * 64,
                          head, m0, batch);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = tc::mbar_wait(kv_full, 0, abort_flag);
      const uint32_t k_addr = tc::smem_u32(s_k), v_addr = tc::smem_u32(s_v);
      const uint32_t p_addr = tc::smem_u32(s_p), ds_addr = tc::smem_u32(s_ds);
      auto issue_s_dp = [&](int it) -> bool {
        const int st = it % kStages;
        if (!tc::mbar_wait(&qdo_full[st], (it / kStages) & 1, abort_flag)) return false;
        if (D == 128 && it > 0 && !tc::mbar_wait(dq_empty, (it - 1) & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t q_addr = tc::smem_u32(s_q + st * kTileBytes);
        const uint32_t do_addr = tc::smem_u32(s_do + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBlkBytes + (kk & 3) * 32;
          tc::umma_f16(tmem_base + kColS, tc::smem_desc(q_addr + off, 16, 1024),
                       tc::smem_desc(k_addr + off, 16, 1024), p.idesc_s, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBlkBytes + (kk & 3) * 32;
          tc::umma_f16(tmem_base + kColDP, tc::smem_desc(do_addr + off, 16, 1024),
                       tc::smem_desc(v_addr + off, 16, 1024), p.idesc_s, kk != 0 ? 1u : 0u);
        }
        tc::umma_commit(sdp_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_s_dp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % kStages;
        if (!tc::mbar_wait(pds_full, it & 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        if constexpr (kPB == 2) {
          // S / dP of the next query block first: the softmax warps have taken block `it` out
          // of tensor memory, and their work on block it + 1 then runs under the three
          // products of block `it` below (which read the other P / dS buffer)
          if (it + 1 < n_iter && !issue_s_dp(it + 1)) { ok = false; break; }
        }
        if (D == 64 && it > 0 && !tc::mbar_wait(dq_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t q_addr = tc::smem_u32(s_q + st * kTileBytes);
        const uint32_t do_addr = tc::smem_u32(s_do + st * kTileBytes);
        const uint32_t pb_addr = p_addr + (it % kPB) * kPdsBytes;
        const uint32_t dsb_addr = ds_addr + (it % kPB) * kPdsBytes;
        // dV += P^T dO ; dK += dS^T Q : A = [q rows x keys] read M-major (M = keys, K = q rows),
        // B = [q rows x D] read N-major.  16 query rows per instruction.
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          const uint64_t b_do = tc::smem_desc(do_addr + kk * 2048, kBlkBytes, 1024);
          const uint64_t b_q = tc::smem_desc(q_addr + kk * 2048, kBlkBytes, 1024);
          const uint64_t a_p = tc::smem_desc(pb_addr + kk * 2048, kBlkBytes, 1024);
          const uint64_t a_ds = tc::smem_desc(dsb_addr + kk * 2048, kBlkBytes, 1024);
          const uint32_t accum = (it | kk) != 0 ? 1u : 0u;
          tc::umma_f16(tmem_base + kColDV, a_p, b_do, p.idesc_dvk, accum);
          tc::umma_f16(tmem_base + kColDK, a_ds, b_q, p.idesc_dvk, accum);
        }
        // dQ_tile = dS K : A = dS K-major (M = q rows, K = keys), B = K read N-major
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          const uint64_t a_ds =
              tc::smem_desc(dsb_addr + (kk >> 2) * kBlkBytes + (kk & 3) * 32, 16, 1024);
          const uint64_t b_k = tc::smem_desc(k_addr + kk * 2048, kBlkBytes, 1024);
          tc::umma_f16(tmem_base + kColDQ, a_ds, b_k, p.idesc_dq, kk != 0 ? 1u : 0u);
        }
        tc::umma_commit(dq_full);
        tc::umma_commit(&qdo_empty[st]);
        if constexpr (kPB == 1) {
          if (it + 1 < n_iter && !issue_s_dp(it + 1)) { ok = false; break; }
        }
      }
      if (ok) tc::umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;   // which 64 of the 128 key columns / which output half
    const int r_in = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    uint64_t seed = 0, offset = 0;
    if (p.p_drop > 0.f) philox_unpack(p.rng, seed, offset);
    const uint32_t add4 = (128u - p.thr7) * 0x01010101u;
    const float keep_prob = 1.f - p.p_drop;
    const float inv_keep = 1.f / keep_prob;
    // dS is formed without the factors scale and 1 / keep_prob; they are applied once to
    // dQ and dK (and 1 / keep_prob to dV) when those leave TMEM
    const float out_scale = p.scale * inv_keep;
    const int sk16 = (p.Sk + 15) >> 4;
    bool ok = true;
    // dQ tile of query block `j`: out of tensor memory into this key tile's fp32 partial.
    // Reductions into one accumulator run at the rate of the L2 atomic units; each key tile
    // stores into its own partial instead (the conversion kernel adds them up).
    auto dq_readout = [&](int j) -> bool {
      if (!tc::mbar_wait_warp(dq_full, j & 1, abort_flag)) return false;
      tc::fence_after_sync();
      const int row = (i_begin + j) * 128 + r_in;
      const bool row_ok = row < p.Sq;
      const bool dq_sliced = p.dq_slice_stride != 0;
      float* dq_dst = p.dq_accum + static_cast<int64_t>(blockIdx.x) * p.dq_slice_stride +
                      ((static_cast<int64_t>(batch) * p.Sq + min(row, p.Sq - 1)) * p.H + head) * p.Dr;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;   // this warp's share of the D columns
        uint32_t r[32];
        tc::tmem_ld_x32(tmem_base + kColDQ + c * 32 + lane_sel, r);
        tc::tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (c * 32 + g * 4 >= p.Dr) break;
            const float4 val = make_float4(__uint_as_float(r[g * 4]) * out_scale,
                                           __uint_as_float(r[g * 4 + 1]) * out_scale,
                                           __uint_as_float(r[g * 4 + 2]) * out_scale,
                                           __uint_as_float(r[g * 4 + 3]) * out_scale);
            if (dq_sliced) *reinterpret_cast<float4*>(dq_dst + c * 32 + g * 4) = val;
            else red_add_v4(dq_dst + c * 32 + g * 4, val.x, val.y, val.z, val.w);
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(dq_empty);
      return true;
    };
    for (int it = 0; it < n_iter && ok; ++it) {
      const int row = (i_begin + it) * 128 + r_in;
      const bool row_ok = row < p.Sq;
      const int64_t stat_idx = (static_cast<int64_t>(batch) * p.H + head) * p.Sq + min(row, p.Sq - 1);
      const float lse2 = row_ok ? p.lse[stat_idx] * kLog2eB : -INFINITY;
      const float delta = row_ok ? p.delta[stat_idx] * keep_prob : 0.f;
      const uint64_t drop_row_base = static_cast<uint64_t>(stat_idx) * sk16;
      const float* rel_row = nullptr;
      float* drel_row = nullptr;
      if (p.rel != nullptr) {
        const int64_t base = static_cast<int64_t>(head) * (p.Sq + p.Sk - 1) + (p.Sq - 1) - min(row, p.Sq - 1);
        rel_row = p.rel + base;
        if (p.drel != nullptr) drel_row = p.drel + base;
      }
      int key_limit = p.Sk;
      if (p.causal) key_limit = min(key_limit, row + diag + 1);
      if (!row_ok || lse2 == -INFINITY) key_limit = 0;
      if (!tc::mbar_wait_warp(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      tc::fence_after_sync();
      uint8_t* p_row = s_p + (it % kPB) * kPdsBytes + r_in * 128;
      uint8_t* ds_row = s_ds + (it % kPB) * kPdsBytes + r_in * 128;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t s_raw[32], dp_raw[32];
        tc::tmem_ld_x32(tmem_base + kColS + c * 32 + lane_sel, s_raw);
        tc::tmem_ld_x32(tmem_base + kColDP + c * 32 + lane_sel, dp_raw);
        tc::tmem_ld_wait();
        float pv[32], dsv[32];
        if constexpr (kPlain) {
#pragma unroll
          for (int t = 0; t < 32; ++t)
            pv[t] = exp2f(fmaf(__uint_as_float(s_raw[t]), p.scale_log2, -lse2));
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int key = n0 + c * 32 + t;
            float s2 = __uint_as_float(s_raw[t]) * p.scale_log2 + kb_tile[c * 32 + t];
            if (rel_row != nullptr) s2 += rel_row[key] * kLog2eB;
            pv[t] = key < key_limit ? exp2f(s2 - lse2) : 0.f;
          }
        }
        if (p.p_drop > 0.f) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 kw = philox_keep16(seed, offset,
                                           drop_row_base + ((n0 + c * 32 + h * 16) >> 4), add4);
            const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int e = h * 16 + i * 4 + j;
                const float pr = pv[e];
                // kept probability (zero where dropped); dS / keep_prob = P (mask dP - delta')
                const float pm = __uint_as_float(__float_as_uint(pr) & keep_mask_full(w[i], j));
                dsv[e] = fmaf(pm, __uint_as_float(dp_raw[e]), -pr * delta);
                pv[e] = pm;
              }
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) dsv[t] = pv[t] * (__uint_as_float(dp_raw[t]) - delta);
        }
        if (drel_row != nullptr) {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int key = n0 + c * 32 + t;
            if (key < key_limit && dsv[t] != 0.f) atomicAdd(drel_row + key, dsv[t] * inv_keep);
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;
          const int off = (c >> 1) * kBlkBytes + ((chunk ^ (r_in & 7)) << 4);
          uint4 pk = make_uint4(pack_pair_b(pv[g * 8 + 0], pv[g * 8 + 1], p.bf16),
                                pack_pair_b(pv[g * 8 + 2], pv[g * 8 + 3], p.bf16),
                                pack_pair_b(pv[g * 8 + 4], pv[g * 8 + 5], p.bf16),
                                pack_pair_b(pv[g * 8 + 6], pv[g * 8 + 7], p.bf16));
          *reinterpret_cast<uint4*>(p_row + off) = pk;
          uint4 dk = make_uint4(pack_pair_b(dsv[g * 8 + 0], dsv[g * 8 + 1], p.bf16),
                                pack_pair_b(dsv[g * 8 + 2], dsv[g * 8 + 3], p.bf16),
                                pack_pair_b(dsv[g * 8 + 4], dsv[g * 8 + 5], p.bf16),
                                pack_pair_b(dsv[g * 8 + 6], dsv[g * 8 + 7], p.bf16));
          *reinterpret_cast<uint4*>(ds_row + off) = dk;
        }
      }
      tc::fence_before_sync();
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(pds_full);
      if constexpr (kPB == 2) {
        // with two P / dS buffers the tensor core is already on S / dP of block it + 1: take
        // the dQ tile of the PREVIOUS block out now, the one of this block after the next
        // block's softmax gradient
        if (it > 0 && !dq_readout(it - 1)) { ok = false; break; }
      } else {
        if (!dq_readout(it)) { ok = false; break; }
      }
    }
    if constexpr (kPB == 2) {
      if (ok && n_iter > 0) ok = dq_readout(n_iter - 1);
    }
    // dK / dV of this key tile: thread = key row
    if (ok && n_iter > 0) ok = tc::mbar_wait_warp(acc_full, 0, abort_flag);
    tc::fence_after_sync();
    const int key = n0 + r_in;
    // tcgen05.ld is warp-collective: every lane takes part, only the stores
    // are predicated on the key being in range
    if (ok) {
      const int key_c = min(key, p.Sk - 1);
      uint8_t* dk_dst = static_cast<uint8_t*>(p.dK) +
                        ((static_cast<int64_t>(batch) * p.Sk + key_c) * p.H + head) * p.dkv_row_stride * 2;
      uint8_t* dv_dst = static_cast<uint8_t*>(p.dV) +
                        ((static_cast<int64_t>(batch) * p.Sk + key_c) * p.H + head) * p.dkv_row_stride * 2;
      {
        // the first four softmax warps write dV, the other four dK
        const int which = half;
        uint8_t* dst = which == 0 ? dv_dst : dk_dst;
        const uint32_t col = which == 0 ? kColDV : kColDK;
        const float f = which == 0 ? inv_keep : out_scale;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          if (n_iter > 0) {
            tc::tmem_ld_x32(tmem_base + col + c * 32 + lane_sel, r);
            tc::tmem_ld_wait();
          } else {
#pragma unroll
            for (int t = 0; t < 32; ++t) r[t] = 0u;
          }
          if (key < p.Sk) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (c * 32 + g * 8 >= p.Dr) break;
              uint4 pk = make_uint4(
                  pack_pair_b(__uint_as_float(r[g * 8 + 0]) * f, __uint_as_float(r[g * 8 + 1]) * f, p.bf16),
                  pack_pair_b(__uint_as_float(r[g * 8 + 2]) * f, __uint_as_float(r[g * 8 + 3]) * f, p.bf16),
                  pack_pair_b(__uint_as_float(r[g * 8 + 4]) * f, __uint_as_float(r[g * 8 + 5]) * f, p.bf16),
                  pack_pair_b(__uint_as_float(r[g * 8 + 6]) * f, __uint_as_float(r[g * 8 + 7]) * f, p.bf16));
              *reinterpret_cast<uint4*>(dst + (c * 32 + g * 8) * 2) = pk;
            }
          }
        }
      }
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 3);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dq (16-bit, rows spaced out_row_stride elements apart) <- sum of the fp32 partials (contiguous
// rows of D, one partial per 128-key tile, slice_stride elements apart; a single accumulator
// when n_slices == 1): the conversion that closes the backward pass; 8 values per thread,
// 16-byte stores.  Under a causal mask key tile kt holds rows of query tiles >= first_q(kt)
// only (the others were never written and are skipped).
template <typename T>
__global__ void __launch_bounds__(256) flash_dq_convert_kernel(
    const float* __restrict__ acc, T* __restrict__ out, int64_t rows, int D, int64_t out_row_stride,
    int n_slices, int64_t slice_stride, int Sq, int Sk, int H, int causal) {
  const int vecs_per_row = D >> 3;
  const int64_t n_vec = rows * vecs_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int diag = Sk - Sq;
  const int q_tiles = (Sq + 127) / 128;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += stride) {
    const int64_t row = i / vecs_per_row;
    const int d = static_cast<int>(i - row * vecs_per_row) * 8;
    const int q_tile = static_cast<int>((row / H) % Sq) >> 7;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int kt = 0; kt < n_slices; ++kt) {
      if (causal && n_slices > 1) {
        int first_q = (kt * 128 - diag) / 128;
        first_q = first_q < 0 ? 0 : (first_q > q_tiles ? q_tiles : first_q);
        if (q_tile < first_q) break;      // later key tiles start even later
      }
      float part[8];
      Vec8<float>::load(acc + kt * slice_stride + row * D + d, part);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += part[j];
    }
    Vec8<T>::store(out + row * out_row_stride + d, v);
  }
}

void launch_flash_dq_convert(const float* acc, void* out, int64_t rows, int D,
                             int64_t out_row_stride, bool bf16, int n_slices, int64_t slice_stride,
                             int Sq, int Sk, int H, int causal, cudaStream_t stream) {
  const int64_t n_vec = rows * (D >> 3);
  if (n_vec == 0) return;
  int64_t blocks = (n_vec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  count_launch();
  if (bf16)
    flash_dq_convert_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(
        acc, static_cast<__nv_bfloat16*>(out), rows, D, out_row_stride, n_slices, slice_stride, Sq,
        Sk, H, causal);
  else
    flash_dq_convert_kernel<__half><<<static_cast<int>(blocks), 256, 0, stream>>>(
        acc, static_cast<__half*>(out), rows, D, out_row_stride, n_slices, slice_stride, Sq, Sk, H,
        causal);
}

template <int D, bool kPlain>
static int launch_bwd_d(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                        const CUtensorMap& tdo, const FlashBwdParams& p, cudaStream_t stream) {
  constexpr int kStages = D == 64 ? 2 : 1;
  constexpr int kPB = D == 64 ? 2 : 1;
  constexpr int kSmem = (2 + 2 * kStages) * 128 * D * 2 + kPB * 4 * 128 * 128 + 12 * 8 + 128 * 4 + 1024;
  static_assert(kSmem <= 227 * 1024, "flash backward: shared memory over the per-CTA limit");
  auto kernel = flash_bwd_kernel<D, kPlain>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess)
      return 3;
    configured = true;
  }
  dim3 grid((p.Sk + 127) / 128, p.H, p.B);
  count_launch();
  kernel<<<grid, 320, kSmem, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int launch_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                     const float* lse, float* delta, float* dq_accum, int64_t dq_slice_stride,
                     void* dk, void* dv, int64_t dkv_row_stride, const float* kbias, const float* rel, float* drel,
                     int B, int H, int Sq, int Sk, int D, const int64_t* q_strides, const int64_t* k_strides,
                     const int64_t* v_strides, float scale, int causal, float p_drop,
                     PhiloxArgs rng, bool bf16, int* status, cudaStream_t stream) {
  if (D < 8 || D > 128 || D % 8 != 0) return 1;
  const int Dt = D <= 64 ? 64 : 128;     // tile width; columns D .. Dt - 1 are zero-filled by TMA
  // pre-pass: delta (o and dout are contiguous [B, Sq, H, D])
  {
    const int64_t rows = static_cast<int64_t>(B) * Sq * H;
    const int wpb = 8;
    const int64_t rows_per_block = static_cast<int64_t>(wpb) * (256 / Dt);
    const unsigned blocks = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
    count_launch();
    if (bf16)
      flash_bwd_delta_kernel<__nv_bfloat16><<<blocks, wpb * 32, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(o), delta, B, H,
          Sq, Dt, D);
    else
      flash_bwd_delta_kernel<__half><<<blocks, wpb * 32, 0, stream>>>(
          static_cast<const __half*>(dout), static_cast<const __half*>(o), delta, B, H, Sq, Dt, D);
  }
  CUtensorMap tq, tk, tv, tdo;
  const int64_t do_strides[3] = {static_cast<int64_t>(Sq) * H * D, static_cast<int64_t>(H) * D, D};
  if (!make_tmap_bshd(&tq, q, B, Sq, H, D, q_strides[0], q_strides[1], q_strides[2], 128, bf16) ||
      !make_tmap_bshd(&tk, k, B, Sk, H, D, k_strides[0], k_strides[1], k_strides[2], 128, bf16) ||
      !make_tmap_bshd(&tv, v, B, Sk, H, D, v_strides[0], v_strides[1], v_strides[2], 128, bf16) ||
      !make_tmap_bshd(&tdo, dout, B, Sq, H, D, do_strides[0], do_strides[1], do_strides[2], 128, bf16))
    return 2;
  FlashBwdParams p;
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.Dr = D; p.lse = lse; p.delta = delta; p.dq_accum = dq_accum;
  p.dq_slice_stride = dq_slice_stride;
  p.dK = dk; p.dV = dv; p.dkv_row_stride = dkv_row_stride; p.kbias = kbias; p.rel = rel; p.drel = drel; p.scale = scale;
  p.scale_log2 = scale * kLog2eB; p.causal = causal; p.rng = rng;
  p.thr7 = dropout_thr7(p_drop);   // same quantisation as the forward kernel
  p.p_drop = p.thr7 / 128.f;
  p.bf16 = bf16 ? 1 : 0; p.status = status;
  const int f = bf16 ? 1 : 0;
  p.idesc_s = tc::instr_desc_f16(128, 128, f, false, false);   // S, dP
  p.idesc_dvk = tc::instr_desc_f16(128, Dt, f, true, true);     // dV, dK
  p.idesc_dq = tc::instr_desc_f16(128, Dt, f, false, true);     // dQ
  const bool plain = kbias == nullptr && rel == nullptr && !causal && Sk % 128 == 0 && Sq % 128 == 0;
  if (Dt == 64)
    return plain ? launch_bwd_d<64, true>(tq, tk, tv, tdo, p, stream)
                 : launch_bwd_d<64, false>(tq, tk, tv, tdo, p, stream);
  return plain ? launch_bwd_d<128, true>(tq, tk, tv, tdo, p, stream)
               : launch_bwd_d<128, false>(tq, tk, tv, tdo, p, stream);
}

}  // namespace slapo
