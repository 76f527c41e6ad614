// Fused GEMM + collective kernels over NVLink peer memory (sm_100a).
//
// One persistent tcgen05 kernel (same pipeline as gemm.cu: TMA producer warp,
// MMA warp, four epilogue warps, TMEM double buffering) extended so that the
// collective which precedes or follows a tensor-parallel GEMM happens inside
// the kernel, tile by tile, while the tensor core keeps working:
//
//   all-gather -> GEMM   an operand is "segmented": segment r lives in rank
//                        r's symmetric buffer and is read in place with TMA
//                        tile loads through a per-peer tensor map (plain tile
//                        loads, this CTA's shared memory only).  Either the
//                        rows of A (forward of a column-parallel layer under
//                        sequence parallelism, dgrad of a row-parallel one) or
//                        the contraction dimension of A or B (weight
//                        gradients, where the gathered tensor is contracted).
//   GEMM -> reduce-scatter   the epilogue writes each 16-bit partial tile into
//                        this rank's symmetric partial buffer.  Tiles are
//                        visited row block by row block: block b of every
//                        owner's rows in turn, then block b + 1.  When a
//                        source has finished a block it raises the block's
//                        flag in its own buffer header, which the owner
//                        polls over NVLink; the owner's reducer warps (warps 6-9 of every CTA,
//                        joined by the epilogue warps once their tiles are
//                        stored) pull the block from all ranks over NVLink
//                        with wide coalesced loads (fp32 sum, optional bias)
//                        and write the result - while the tensor core works
//                        on the later blocks.  Once a CTA's main loop is over
//                        the pulled vectors are parked in the operand
//                        pipeline's shared memory (asynchronous copies, 192
//                        KB per SM on the wire) instead of in registers.
//   GEMM -> all-reduce   reduce-scatter as above, the reduced rows go to
//                        every peer's output buffer and a second flag round
//                        closes the operation.
//
// Both transfers spread over all peers at once: the gather's copy units are taken block by
// block across owners (a CTA pulls block b of owner o while its neighbour pulls block b of
// owner o + 1), and the reduction reads a vector from every source together.  Peer by peer
// - every GPU reading from exactly one other GPU at a time - measured half the bandwidth
// of the spread pattern on an 8-GPU NVSwitch node.
//
// With an NVLS address of the partial-product buffers (`mc_recv`, the same symmetric buffer
// bound to an NVSwitch group) the reduction issues ONE `multimem.ld_reduce` per 16 bytes: the
// switch fetches and adds the eight ranks' vectors (fp32 accumulation) and a tenth of the
// loads in flight reaches the link rate, so the reducer warps alone keep NVLink busy while
// the main loop still runs; the all-reduce's second half is one `multimem.st` per vector.
// The peer-load path stays for groups without such an address (and for tests where a rank
// may leave: a rank must not die while bound to a switch group).
//
// Flow control is an int32 flag pad in symmetric memory and one job-wide
// monotone epoch number per fused operation (identical on all ranks):
//   ready[src] >= epoch   rank src has entered this operation, i.e. everything
//                         it launched before (producers of its buffers,
//                         consumers of what we are about to overwrite) is done
//   blk[m] >= epoch       (header of rank src's partial buffer) src has stored row block m
//   done2[src] >= epoch   rank src has delivered its reduced rows (all-reduce)
// Every wait is bounded; on time-out the kernel records an error code in the
// device status word, stops issuing work and leaves (TMEM freed).
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace slapo {

constexpr int kMaxRanks = 8;
// the chunk_flags argument points at 2 * kChunkCountOffset words: ready flags of the staged row
// blocks first, slice counters of the same blocks behind them
constexpr int kChunkCountOffset = 8192;
// header of a partial-product (receive) buffer: kChunkCountOffset block flags + as many counters
constexpr int kRecvHeaderBytes = 2 * kChunkCountOffset * 4;
// pushed gather: flag words per 128-row block in the slot header (one per slice, up to 16)
constexpr int kSliceFlagStride = 16;
constexpr int kDefaultAgSlices = 1;
constexpr int kDefaultAgInflight = 16;
constexpr int CBM = 128;
constexpr int CBK = 64;

struct SegMaps {
  CUtensorMap map[kMaxRanks];
};

enum CommMode { kModeLocal = 0, kModeReduceScatter = 1, kModeAllReduce = 2 };

struct CommGemmParams {
  int M, N, K;
  int world, rank;
  // operand gathering: 0 none, 1 rows of A (M), 2 contraction dim of A, 3 contraction dim of B
  int gather;
  int seg_len;          // extent of one rank's segment along the gathered dimension
  int mode;
  int epoch;
  // local output (kModeLocal) or reduced output [M / world, N] (reduce-scatter) or [M, N] (all-reduce)
  void* out;
  int ldo;
  const void* bias;     // added after the reduction (or in the plain epilogue)
  int act;
  int bf16;
  uint32_t idesc;
  // symmetric state
  int* flags;                    // local pad: ready[8] | done[8] | done2[8] | counters[8]
  int* peer_flags[kMaxRanks];    // the same pad on every rank
  void* peer_recv[kMaxRanks];    // every rank's partial-product buffer [M, N] 16-bit
  void* peer_out[kMaxRanks];     // all-reduce output buffers [M, N]
  int* status;
  long long wait_cycles;         // budget of a cross-GPU wait
  // gather mode 4 (rows of A staged through local memory)
  void* stage_dst;               // local [M, K] buffer the copier warps fill
  int* chunk_flags;              // local, one word per 128-row block: epoch when staged
  const void* seg_src[kMaxRanks];  // every rank's shard [seg_len, K]
  int row_bytes;                 // K * 2
  int trace;                     // record phase time stamps (debug aid)
  int ag_slices;                 // staged gather: slices per 128-row block (1, 2 or 4)
  int ag_inflight;               // staged gather: 16-byte loads in flight per thread (8 or 16)
  // reduce-scatter / all-reduce: the header of every rank's partial-product buffer holds one
  // flag per 128-row block of that buffer (epoch when all its tiles were stored; owners poll the
  // flags of their rows in every rank's header) and the local arrival counters
  int* blk_flags;
  int* peer_blk_flags[kMaxRanks];
  int* blk_counters;
  // NVLS addresses (null = peer loads / stores): the partial-product buffers of all ranks
  // behind one address (header first), and the all-reduce output buffers
  int* mc_blk_flags;
  void* mc_recv;
  void* mc_out;
  // gather mode 5 (rows of A pushed by their owners): every rank's staging slot [M, K] and the
  // block flags in the slot's header; `mc_stage` is the slots of all ranks behind one
  // multicast address (null: one store per rank)
  void* peer_stage[kMaxRanks];
  int* peer_chunk_flags[kMaxRanks];
  void* mc_stage;
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Phase trace, a debugging aid (off unless SLAPO_B200_COMM_TRACE=1): every CTA of the last fused
// kernel records the nanosecond timer at a few points; `read_comm_trace` copies the table out.
//   0 kernel entry   1 copier / reducer: first unit starts   2 copier / reducer: last unit done
//   3 producer: first wait for a staged block begins   4 ... ends   5 epilogue: last tile stored
//   6 kernel exit    7 producer: nanoseconds spent waiting for staged blocks
constexpr int kTraceSlots = 8;
constexpr int kTraceCtas = 256;
__device__ unsigned long long g_comm_trace[kTraceCtas * kTraceSlots];
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_mark(int on, int slot) {
  if (on && blockIdx.x < kTraceCtas) g_comm_trace[blockIdx.x * kTraceSlots + slot] = gtimer();
}

// Debug build (`SLAPO_B200_DEBUG=1 python -m slapo_b200.csrc.build -f`): every index that
// becomes a peer address or a flag slot is checked first; a violation records status 7 and
// the access is skipped instead of faulting another GPU's memory.
#ifdef SLAPO_B200_DEBUG
#define SLAPO_DBG_CHECK(cond, status_ptr)                                       \
  if (!(cond)) {                                                                \
    if ((status_ptr) != nullptr) atomicExch((status_ptr), 7);                   \
    continue;                                                                   \
  }
#else
#define SLAPO_DBG_CHECK(cond, status_ptr)
#endif

// bounded spin on a flag written by another GPU
__device__ __forceinline__ bool wait_flag(const int* addr, int epoch, long long budget,
                                          volatile int* abort_flag) {
  if (ld_acquire_sys(addr) >= epoch) return true;
  const long long start = clock64();
  int spins = 0;
  while (ld_acquire_sys(addr) < epoch) {
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > budget) {
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}

// bounded wait for the first `n` flag words of a 16-word group (the slices of one 128-row block
// of the pushed gather), polled with 16-byte loads; ends with the acquiring fence
__device__ __forceinline__ bool wait_flags16(const int* addr, int n, int epoch, long long budget,
                                             volatile int* abort_flag) {
  const long long start = clock64();
  int spins = 0;
  for (;;) {
    bool all = true;
    for (int i = 0; i < n; i += 4) {
      int4 v;
      asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr + i) : "memory");
      all = all && v.x >= epoch && (i + 1 >= n || v.y >= epoch) && (i + 2 >= n || v.z >= epoch) &&
            (i + 3 >= n || v.w >= epoch);
    }
    if (all) break;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > budget) {
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(64);
  }
  __threadfence_system();
  return true;
}

// all NT threads of the copier / reducer group agree on a predicate computed by its first thread
template <int NT = 128>
__device__ __forceinline__ int __syncthreads_or_named(int v) {
  __shared__ int s_copier_vote;
  if (threadIdx.x == 192) s_copier_vote = v;
  asm volatile("bar.sync 2, %0;" ::"n"(NT) : "memory");
  const int r = s_copier_vote;
  asm volatile("bar.sync 2, %0;" ::"n"(NT) : "memory");
  return r;
}

template <int BN, int STAGES>
struct CommSmem {
  static constexpr int kABytes = CBM * CBK * 2;
  static constexpr int kBBytes = BN * CBK * 2;
  static constexpr int kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kTotal = kBarOffset + 256 + 1024;
  // after the main loop the reduction parks pulled vectors in the pipeline's memory (2 x 96 KB)
  static_assert(kBarOffset >= 192 * 1024, "operand pipeline smaller than the reduction's staging area");
};

__device__ __forceinline__ uint32_t cpack2(float a, float b, int bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float cload(const void* p, int64_t i, int bf16) {
  if (bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

// Tile order.  Gather: row blocks are visited owner by owner, own rows first (first = 0), remote
// rows while they are being staged.  Scatter (interleave): the b-th row block of every owner in
// turn, starting with the rank after this one, then block b + 1 - so that block b of an owner is
// complete on ALL ranks after (b + 1) / blocks_per_owner of the main loop and its reduction
// overlaps the rest of the GEMM.
__device__ __forceinline__ void tile_coords(int t, int tiles_n, int blocks_per_owner, int world,
                                            int rank, bool rotate, int& m_blk, int& n_blk,
                                            int first = 1, bool interleave = false,
                                            bool own_then_spread = false) {
  n_blk = t % tiles_n;
  int mb = t / tiles_n;
  if (rotate) {
    int o_idx, b;
    if (own_then_spread) {
      // staged gather: this rank's blocks, then block b of every other owner in turn - the
      // order in which the copier warps of all CTAs bring them in
      if (mb < blocks_per_owner) {
        o_idx = 0;
        b = mb;
      } else {
        const int idx = mb - blocks_per_owner;
        b = idx / (world - 1);
        o_idx = 1 + idx % (world - 1);
      }
    } else if (interleave) {
      o_idx = mb % world;
      b = mb / world;
    } else {
      o_idx = mb / blocks_per_owner;
      b = mb % blocks_per_owner;
    }
    const int owner = (rank + first + o_idx) % world;
    mb = owner * blocks_per_owner + b;
  }
  m_blk = mb;
}

// Reduction phase of GEMM -> reduce-scatter / all-reduce: this rank sums its rows of every
// rank's partial-product buffer (16-byte coalesced peer loads), adds bias / activation and
// writes the result (to every rank's output for all-reduce).  W = group size known at compile
// time (0 = generic), U = row vectors per thread per iteration: W * U loads are in flight per
// thread before the first is used, which is what hides the NVLink round trip.
template <int W, int U>
__device__ __forceinline__ void reduce_span(const CommGemmParams& p, int rows_per_rank, int row0,
                                            int nrows, int tid, int nthr) {
  // rows [row0, row0 + nrows) of this rank's [rows_per_rank, N] rows; 32-bit indices inside the span
  constexpr int kW = W > 0 ? W : kMaxRanks;
  const int world = W > 0 ? W : p.world;
  const unsigned vpr = static_cast<unsigned>(p.N) / 8u;     // 8-element vectors per row
  const unsigned n_loc = static_cast<unsigned>(nrows) * vpr;
  // this rank's rows inside every source's partial buffer [M, N]
  const int64_t my_off = (static_cast<int64_t>(p.rank) * rows_per_rank + row0) * p.N;
  const uint8_t* srcs[kW];
#pragma unroll
  for (int r = 0; r < kW; ++r) {
    // start with the next rank so that the peers' links share the load
    int src = p.rank + 1 + r;
    if (src >= world) src -= world;
    srcs[r] = r < world ? static_cast<const uint8_t*>(p.peer_recv[src]) + my_off * 2 : nullptr;
  }
  for (unsigned j0 = tid; j0 < n_loc; j0 += static_cast<unsigned>(nthr) * U) {
    uint4 raw[U][kW];
    if constexpr (W > 0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned j = j0 + u * nthr;
#pragma unroll
        for (int r = 0; r < kW; ++r)
          if (j < n_loc)
            raw[u][r] = __ldcg(reinterpret_cast<const uint4*>(srcs[r] + static_cast<size_t>(j) * 16));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned j = j0 + u * nthr;
      if (j >= n_loc) break;
      float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kW; ++r) {
        if (r < world) {
          float v[8];
          // group sizes without an instantiation (3, 5, 6, 7) load source by source
          if constexpr (W == 0)
            raw[u][r] = __ldcg(reinterpret_cast<const uint4*>(srcs[r] + static_cast<size_t>(j) * 16));
          if (p.bf16) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][r]);
#pragma unroll
            for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
          } else {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[u][r]);
#pragma unroll
            for (int k = 0; k < 4; ++k) { float2 f = __half22float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) acc8[k] += v[k];
        }
      }
      const unsigned lr = j / vpr;
      const int col = static_cast<int>(j - lr * vpr) * 8;
      if (p.bias != nullptr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc8[k] += cload(p.bias, col + k, p.bf16);
      }
      if (p.act >= 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc8[k] = act_fwd(acc8[k], p.act);
      }
      const int64_t lrow = row0 + static_cast<int>(lr);
      if (p.mode == kModeReduceScatter) {
        void* o = static_cast<uint8_t*>(p.out) + (lrow * p.ldo + col) * 2;
        if (p.bf16) Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(o), acc8);
        else Vec8<__half>::store(static_cast<__half*>(o), acc8);
      } else {
        // all-reduce: the reduced rows go to every rank's output buffer
        const int64_t grow = static_cast<int64_t>(p.rank) * rows_per_rank + lrow;
        for (int r = 0; r < world; ++r) {
          int peer = p.rank + r;
          if (peer >= world) peer -= world;
          void* o = static_cast<uint8_t*>(p.peer_out[peer]) + (grow * p.ldo + col) * 2;
          if (p.bf16) Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(o), acc8);
          else Vec8<__half>::store(static_cast<__half*>(o), acc8);
        }
      }
    }
  }
}

// The same reduction with the pulled vectors parked in shared memory instead of registers, for
// the time after the main loop when the operand pipeline's 192 KB are free: every thread of a
// 128-thread group owns 768 bytes of the group's 96 KB and fills them with 48 asynchronous
// 16-byte copies (48 / W vectors from each of the W sources) before it waits - 96 KB per group on
// the wire instead of the 32 KB that registers hold, which turns the pull from round-trip-bound
// into bandwidth-bound.  A thread only reads back what it copied itself, so the copies need no
// barrier.  `region` = shared-memory address of the group's 96 KB.
template <int W>
__device__ __forceinline__ void reduce_span_smem(const CommGemmParams& p, int rows_per_rank,
                                                 int row0, int nrows, int gt, uint32_t region) {
  constexpr int U = 48 / W;
  const unsigned vpr = static_cast<unsigned>(p.N) / 8u;
  const unsigned n_loc = static_cast<unsigned>(nrows) * vpr;
  const int64_t my_off = (static_cast<int64_t>(p.rank) * rows_per_rank + row0) * p.N;
  const uint8_t* srcs[W];
#pragma unroll
  for (int r = 0; r < W; ++r) {
    int src = p.rank + 1 + r;
    if (src >= W) src -= W;
    srcs[r] = static_cast<const uint8_t*>(p.peer_recv[src]) + my_off * 2;
  }
  const uint32_t mine = region + static_cast<uint32_t>(gt) * 16u;   // slot (u, r) at + (u * W + r) * 2048
  for (unsigned j0 = gt; j0 < n_loc; j0 += 128u * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned j = j0 + u * 128u;
      if (j < n_loc) {
#pragma unroll
        for (int r = 0; r < W; ++r)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mine + (u * W + r) * 2048u),
                       "l"(srcs[r] + static_cast<size_t>(j) * 16)
                       : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll 2
    for (int u = 0; u < U; ++u) {
      const unsigned j = j0 + u * 128u;
      if (j >= n_loc) break;
      float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < W; ++r) {
        uint4 raw;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "r"(mine + (u * W + r) * 2048u));
        float v[8];
        if (p.bf16) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
        } else {
          const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
          for (int k = 0; k < 4; ++k) { float2 f = __half22float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) acc8[k] += v[k];
      }
      const unsigned lr = j / vpr;
      const int col = static_cast<int>(j - lr * vpr) * 8;
      if (p.bias != nullptr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc8[k] += cload(p.bias, col + k, p.bf16);
      }
      if (p.act >= 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc8[k] = act_fwd(acc8[k], p.act);
      }
      const int64_t lrow = row0 + static_cast<int>(lr);
      if (p.mode == kModeReduceScatter) {
        void* o = static_cast<uint8_t*>(p.out) + (lrow * p.ldo + col) * 2;
        if (p.bf16) Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(o), acc8);
        else Vec8<__half>::store(static_cast<__half*>(o), acc8);
      } else {
        const int64_t grow = static_cast<int64_t>(p.rank) * rows_per_rank + lrow;
        for (int r = 0; r < W; ++r) {
          int peer = p.rank + r;
          if (peer >= W) peer -= W;
          void* o = static_cast<uint8_t*>(p.peer_out[peer]) + (grow * p.ldo + col) * 2;
          if (p.bf16) Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(o), acc8);
          else Vec8<__half>::store(static_cast<__half*>(o), acc8);
        }
      }
    }
  }
}


// ---- NVLS (multimem) -------------------------------------------------------
// one load returns the sum over all ranks of the 16-byte vector at this address
__device__ __forceinline__ uint4 mc_ld_reduce_add(const void* mc_addr, int bf16) {
  uint4 v;
  if (bf16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
// the smallest value that any rank holds in this flag word
__device__ __forceinline__ int mc_ld_min_acquire(const int* mc_addr) {
  int v;
  asm volatile("multimem.ld_reduce.acquire.sys.global.min.s32 %0, [%1];" : "=r"(v) : "l"(mc_addr) : "memory");
  return v;
}
// one store lands in every rank's copy of the buffer
__device__ __forceinline__ void mc_st(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ bool wait_flag_mc(const int* mc_addr, int epoch, long long budget,
                                             volatile int* abort_flag) {
  if (mc_ld_min_acquire(mc_addr) >= epoch) return true;
  const long long start = clock64();
  int spins = 0;
  while (mc_ld_min_acquire(mc_addr) < epoch) {
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > budget) {
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}

// The reduction through the switch: U loads in flight per thread, each already the fp32-
// accumulated sum over the group rounded to the 16-bit type; bias / activation follow.
template <int U>
__device__ __forceinline__ void reduce_span_mc(const CommGemmParams& p, int rows_per_rank,
                                               int row0, int nrows, int tid, int nthr) {
  const unsigned vpr = static_cast<unsigned>(p.N) / 8u;
  const unsigned n_loc = static_cast<unsigned>(nrows) * vpr;
  const int64_t my_off = (static_cast<int64_t>(p.rank) * rows_per_rank + row0) * p.N;
  const uint8_t* src = static_cast<const uint8_t*>(p.mc_recv) + my_off * 2;
  for (unsigned j0 = tid; j0 < n_loc; j0 += static_cast<unsigned>(nthr) * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned j = j0 + u * nthr;
      if (j < n_loc) raw[u] = mc_ld_reduce_add(src + static_cast<size_t>(j) * 16, p.bf16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned j = j0 + u * nthr;
      if (j >= n_loc) break;
      const unsigned lr = j / vpr;
      const int col = static_cast<int>(j - lr * vpr) * 8;
      uint4 outv = raw[u];
      if (p.bias != nullptr || p.act >= 0) {
        float v[8];
        if (p.bf16) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
          for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
        } else {
          const __half2* h = reinterpret_cast<const __half2*>(&raw[u]);
#pragma unroll
          for (int k = 0; k < 4; ++k) { float2 f = __half22float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] += cload(p.bias, col + k, p.bf16);
        }
        if (p.act >= 0) {
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = act_fwd(v[k], p.act);
        }
        outv = make_uint4(cpack2(v[0], v[1], p.bf16), cpack2(v[2], v[3], p.bf16),
                          cpack2(v[4], v[5], p.bf16), cpack2(v[6], v[7], p.bf16));
      }
      const int64_t lrow = row0 + static_cast<int>(lr);
      if (p.mode == kModeReduceScatter) {
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + (lrow * p.ldo + col) * 2) = outv;
      } else {
        const int64_t grow = static_cast<int64_t>(p.rank) * rows_per_rank + lrow;
        if (p.mc_out != nullptr) {
          mc_st(static_cast<uint8_t*>(p.mc_out) + (grow * p.ldo + col) * 2, outv);
        } else {
          for (int r = 0; r < p.world; ++r)
            *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peer_out[r]) +
                                      (grow * p.ldo + col) * 2) = outv;
        }
      }
    }
  }
}

// One group of 128 threads (named barrier `bar_id`, `gt` = thread index inside the group) takes
// reduction units of this CTA until none is left.  A unit is a 32-row slice of a 128-row block of
// this rank's rows; the reducer warps (from the start) and the epilogue warps (once their tiles
// are done) of all CTAs share the units.  A unit is reduced when the block's
// flags from every source rank have arrived.
__device__ __forceinline__ void reduce_units(const CommGemmParams& p, int rows_per_rank,
                                             int blocks_per_owner, int gt, int bar_id, int* next_k,
                                             volatile int* vote, volatile int* abort_flag,
                                             volatile int* pipe_free, uint32_t region) {
  constexpr int kRedSlices = 4;
  const int units = blocks_per_owner * kRedSlices;
  for (;;) {
    if (gt == 0) {
      // units are handed out in block order by one counter for the whole GPU (word 40 of the
      // flag pad, reset by the last CTA to leave): whichever group is free takes the lowest
      // outstanding unit, so that no CTA is left with an extra unit at the end
      (void)next_k;
      const int u = atomicAdd(p.flags + 40, 1);
      vote[0] = u;
      vote[1] = *abort_flag != 0 ? 0 : (u < units ? 1 : -1);   // 0 stop (error), -1 no unit left
      vote[2] = *pipe_free;   // the main loop of this CTA is over: its shared memory is free
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    const int u = vote[0];
    if (vote[1] == 1 && p.mc_blk_flags != nullptr) {
      // one load through the switch returns the minimum of the block's flag over all ranks
      if (gt == 0 && !wait_flag_mc(p.mc_blk_flags + p.rank * blocks_per_owner + u / kRedSlices,
                                   p.epoch, p.wait_cycles, abort_flag))
        vote[1] = 0;
    } else if (vote[1] == 1 && gt < p.world) {
      // flag of block b of this rank's rows in every source's header (a word of the peer's
      // memory, polled over NVLink): one thread per source, so the round trips overlap
      const int src = (p.rank + 1 + gt) % p.world;
      if (!wait_flag(p.peer_blk_flags[src] + p.rank * blocks_per_owner + u / kRedSlices, p.epoch,
                     p.wait_cycles, abort_flag))
        vote[1] = 0;
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    const int w = vote[1];
    const int in_smem = vote[2];
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (w != 1) break;
    const int row0 = (u / kRedSlices) * CBM + (u % kRedSlices) * (CBM / kRedSlices);
    SLAPO_DBG_CHECK(row0 + CBM / kRedSlices <= rows_per_rank &&
                        p.rank * blocks_per_owner + u / kRedSlices < kChunkCountOffset,
                    p.status)
    if (p.mc_recv != nullptr) {
      reduce_span_mc<8>(p, rows_per_rank, row0, CBM / kRedSlices, gt, 128);
      continue;
    }
    if (in_smem && (p.world == 2 || p.world == 4 || p.world == 8)) {
      if (p.world == 2) reduce_span_smem<2>(p, rows_per_rank, row0, CBM / kRedSlices, gt, region);
      else if (p.world == 4) reduce_span_smem<4>(p, rows_per_rank, row0, CBM / kRedSlices, gt, region);
      else reduce_span_smem<8>(p, rows_per_rank, row0, CBM / kRedSlices, gt, region);
      continue;
    }
    switch (p.world) {
      case 2: reduce_span<2, 8>(p, rows_per_rank, row0, CBM / kRedSlices, gt, 128); break;
      case 4: reduce_span<4, 4>(p, rows_per_rank, row0, CBM / kRedSlices, gt, 128); break;
      case 8: reduce_span<8, 2>(p, rows_per_rank, row0, CBM / kRedSlices, gt, 128); break;
      default: reduce_span<0, 1>(p, rows_per_rank, row0, CBM / kRedSlices, gt, 128); break;
    }
  }
}

// NT threads copy n_vec 16-byte vectors, F loads in flight per thread
template <int F, int NT>
__device__ __forceinline__ void copy_vecs(const uint4* src, uint4* dst, int64_t n_vec, int ct) {
  for (int64_t v = ct; v < n_vec; v += NT * F) {
    uint4 tmp[F];
#pragma unroll
    for (int q = 0; q < F; ++q)
      if (v + q * NT < n_vec) tmp[q] = __ldcg(src + v + q * NT);
#pragma unroll
    for (int q = 0; q < F; ++q)
      if (v + q * NT < n_vec) dst[v + q * NT] = tmp[q];
  }
}

// One warp pushes n_vec 16-byte vectors of this rank's shard into the staging slots of all
// ranks at byte offset dst_off: through the switch (one multicast store) or rank by rank.
// F local loads are in flight per lane; the stores need no answer.
template <int F>
__device__ __forceinline__ void push_vecs(const CommGemmParams& p, const uint4* src,
                                          int64_t dst_off, int n_vec, int lane) {
  for (int v = lane; v < n_vec; v += 32 * F) {
    uint4 tmp[F];
#pragma unroll
    for (int q = 0; q < F; ++q)
      if (v + q * 32 < n_vec) tmp[q] = __ldcg(src + v + q * 32);
    if (p.mc_stage != nullptr) {
#pragma unroll
      for (int q = 0; q < F; ++q)
        if (v + q * 32 < n_vec)
          mc_st(static_cast<uint8_t*>(p.mc_stage) + dst_off + static_cast<int64_t>(v + q * 32) * 16,
                tmp[q]);
    } else {
      for (int rr = 0; rr < p.world; ++rr) {
        int r = p.rank + 1 + rr;             // the other ranks first, this rank's own slot last
        if (r >= p.world) r -= p.world;
        uint8_t* dst = static_cast<uint8_t*>(p.peer_stage[r]) + dst_off;
#pragma unroll
        for (int q = 0; q < F; ++q)
          if (v + q * 32 < n_vec)
            *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(v + q * 32) * 16) = tmp[q];
      }
    }
  }
}

// CW: warps 6 .. 5 + CW are the copier (staged gather, CW = 8) or reducer (scatter modes, CW = 4)
// warps; kernels without either are launched with the first six warps only.
template <int BN, int STAGES, bool A_MN, bool B_MN, int CW>
__global__ void __launch_bounds__(192 + CW * 32, 1)
comm_gemm_kernel(const __grid_constant__ SegMaps maps_a, const __grid_constant__ SegMaps maps_b,
                 const CommGemmParams p) {
  using S = CommSmem<BN, STAGES>;
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
  __shared__ int s_red_next;          // next reduction unit of this CTA (scatter modes)
  __shared__ int s_red_vote[2][4];    // per reducing group: unit, go / stop, pipeline memory free
  __shared__ int s_pipe_free;         // the main loop is over, the operand pipeline's memory is free

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + CBM - 1) / CBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + CBK - 1) / CBK;
  // a role that waits (through an mbarrier) behind another role's wait for a peer GPU must
  // outlast that wait
  const long long mbar_budget = p.wait_cycles + tc::kWaitCycles;
  const bool scatter = p.mode != kModeLocal;
  const int rows_per_rank = p.M / p.world;               // used when rows are owned (gather 1 / scatter)
  const bool pushed = p.gather == 5;
  const bool staged = p.gather == 4 || pushed;
  const int first = staged ? 0 : 1;
  const bool rotate = p.world > 1 && (scatter || p.gather == 1 || staged) && rows_per_rank % CBM == 0;
  const int blocks_per_owner = rotate ? rows_per_rank / CBM : tiles_m;
  constexpr uint32_t kTmemCols = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);

  int* ready = p.flags;
  int* done = p.flags + 8;
  int* done2 = p.flags + 16;
  int* counters = p.flags + 24;

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
    s_red_next = 0;
    s_pipe_free = 0;
    tc::fence_barrier_init();
    trace_mark(p.trace, 0);
    if (p.trace && blockIdx.x < kTraceCtas) g_comm_trace[blockIdx.x * kTraceSlots + 7] = 0;
    // announce: this rank has entered operation `epoch`
    if (blockIdx.x == 0 && p.world > 1) {
      for (int r = 0; r < p.world; ++r) st_release_sys(p.peer_flags[r] + p.rank, p.epoch);
    }
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
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t seen_ready = 1u << p.rank;  // peers whose ready flag has been observed
      bool traced_first = false;
      auto need_ready = [&](int r) -> bool {
        if (seen_ready & (1u << r)) return true;
        if (!wait_flag(ready + r, p.epoch, p.wait_cycles, abort_flag)) return false;
        // order the flag observation before the TMA engine's reads of that peer
        asm volatile("fence.proxy.async;" ::: "memory");
        seen_ready |= 1u << r;
        return true;
      };
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, tiles_n, blocks_per_owner, p.world, p.rank, rotate, m_blk, n_blk, first,
                    scatter, staged);
        const int m0 = m_blk * CBM, n0 = n_blk * BN;
        int a_seg = 0, a_row = m0;
        if (p.gather == 1) {
          a_seg = m0 / p.seg_len;
          a_row = m0 - a_seg * p.seg_len;
          if (!need_ready(a_seg)) { ok = false; break; }
        } else if (staged) {
          if (m0 / p.seg_len == p.rank) {
            a_seg = 0;                      // own shard, read in place
            a_row = m0 - p.rank * p.seg_len;
          } else {
            a_seg = 1;                      // staged copy in local memory
            unsigned long long t_wait = 0;
            if (p.trace) {
              t_wait = gtimer();
              if (!traced_first) g_comm_trace[(blockIdx.x % kTraceCtas) * kTraceSlots + 3] = t_wait;
            }
            const bool arrived =
                pushed ? wait_flags16(p.chunk_flags + m_blk * kSliceFlagStride, p.ag_slices, p.epoch,
                                      p.wait_cycles, abort_flag)
                       : wait_flag(p.chunk_flags + m_blk, p.epoch, p.wait_cycles, abort_flag);
            if (!arrived) {
              ok = false;
              break;
            }
            if (p.trace) {
              const unsigned long long t_end = gtimer();
              if (!traced_first) g_comm_trace[(blockIdx.x % kTraceCtas) * kTraceSlots + 4] = t_end;
              g_comm_trace[(blockIdx.x % kTraceCtas) * kTraceSlots + 7] += t_end - t_wait;
              traced_first = true;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          int k_a = kb * CBK, k_b = kb * CBK, seg_a = a_seg, seg_b = 0;
          if (p.gather == 2) {
            seg_a = k_a / p.seg_len;
            k_a -= seg_a * p.seg_len;
            if (!need_ready(seg_a)) { ok = false; break; }
          } else if (p.gather == 3) {
            seg_b = k_b / p.seg_len;
            k_b -= seg_b * p.seg_len;
            if (!need_ready(seg_b)) { ok = false; break; }
          }
          if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, mbar_budget)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(&full_bar[stage], S::kABytes + S::kBBytes);
          uint8_t* sa = smem_a + stage * S::kABytes;
          uint8_t* sb = smem_b + stage * S::kBBytes;
          const CUtensorMap* ta = &maps_a.map[seg_a];
          const CUtensorMap* tb = &maps_b.map[seg_b];
          if constexpr (!A_MN) {
            tc::tma_load_2d(sa, ta, &full_bar[stage], k_a, a_row);
          } else {
#pragma unroll
            for (int j = 0; j < CBM / 64; ++j)
              tc::tma_load_2d(sa + j * (CBK * 128), ta, &full_bar[stage], a_row + j * 64, k_a);
          }
          if constexpr (!B_MN) {
            tc::tma_load_2d(sb, tb, &full_bar[stage], k_b, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tc::tma_load_2d(sb + j * (CBK * 128), tb, &full_bar[stage], n0 + j * 64, k_b);
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!tc::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, mbar_budget)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&full_bar[stage], phase, abort_flag, mbar_budget)) { ok = false; break; }
          tc::fence_after_sync();
          const uint32_t a_addr = tc::smem_u32(smem_a + stage * S::kABytes);
          const uint32_t b_addr = tc::smem_u32(smem_b + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < CBK / 16; ++k) {
            const uint64_t a_desc = A_MN ? tc::smem_desc(a_addr + k * 2048, CBK * 128, 1024)
                                         : tc::smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t b_desc = B_MN ? tc::smem_desc(b_addr + k * 2048, CBK * 128, 1024)
                                         : tc::smem_desc(b_addr + k * 32, 16, 1024);
            tc::umma_f16(d_tmem, a_desc, b_desc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc::umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc::umma_commit(&tmem_full[acc]);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ copier warps --------------------------------
    // Remote shards cross NVLink exactly once: 128-row blocks are pulled into
    // the local staging buffer (16-byte coalesced loads, 8 in flight per
    // thread) and published block by block; the producer warps of all CTAs
    // read staged blocks with local TMA loads.
    if (pushed && p.world > 1) {
      // Pushed gather.  Copier warps 0 .. CW - 2 are senders: each takes 128 / slices-row
      // slices of this rank's OWN shard in row order (local loads) and stores them into the
      // staging slots of all ranks - one multicast store through the switch, or one store
      // per rank.  Stores need no answer, so a sender never waits for an NVLink round trip:
      // it hands the slice to the publisher through shared memory and goes on; the link's
      // back pressure paces the senders, and because slices go out in row order they also
      // arrive in row order.  The last copier warp is the publisher: whenever senders have
      // handed over new slices it runs ONE system-scope fence - which, being cumulative,
      // covers the senders' stores that it observed through shared memory - and then raises
      // the flag of every covered slice on every rank.  (A fence per slice in the sending
      // warp measured 50 us of stall per round at 8 GPUs.)  The main loops of all ranks wait
      // for the `slices` flags of a 128-row block.
      const int cw = warp - 6;
      constexpr int kSenders = CW - 1;
      __shared__ int s_issued[CW];       // slices handed over by each sender; [CW - 1]: senders done
      const int slices = p.ag_slices;
      const int slice_rows = CBM / slices;
      const int slice_vec = slice_rows * (p.row_bytes / 16);
      const int units = blocks_per_owner * slices;
      const int stride = static_cast<int>(gridDim.x) * kSenders;
      if (cw == 0 && lane < CW) s_issued[lane] = 0;
      asm volatile("bar.sync 2, %0;" ::"n"(CW * 32) : "memory");
      if (cw < kSenders) {
        // Nobody's slot may be written before its owner has entered this operation: its
        // earlier kernels, which read the slot's previous contents, are complete by then.
        int entered = 1;
        if (lane < p.world && lane != p.rank)
          entered = wait_flag(ready + lane, p.epoch, p.wait_cycles, abort_flag) ? 1 : 0;
        const bool ok = __all_sync(0xffffffffu, entered) != 0;
        if (cw == 0 && lane == 0) trace_mark(p.trace, 1);
        int k = 0;
        for (int u = cw * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
             u < units && ok; u += stride, ++k) {
          const int b = u / slices, sl = u - b * slices;
          const int64_t off = (static_cast<int64_t>(b) * CBM + sl * slice_rows) * p.row_bytes;
          SLAPO_DBG_CHECK(off + static_cast<int64_t>(slice_rows) * p.row_bytes <=
                                  static_cast<int64_t>(p.seg_len) * p.row_bytes && (off & 15) == 0,
                          p.status)
          const uint4* src = reinterpret_cast<const uint4*>(
              static_cast<const uint8_t*>(p.seg_src[p.rank]) + off);
          const int64_t dst_off = static_cast<int64_t>(p.rank) * p.seg_len * p.row_bytes + off;
          if (p.ag_inflight == 16) push_vecs<16>(p, src, dst_off, slice_vec, lane);
          else push_vecs<8>(p, src, dst_off, slice_vec, lane);
          __syncwarp();
          if (lane == 0) {
            __threadfence_block();      // release at CTA scope: the hand-over below follows the stores
            *reinterpret_cast<volatile int*>(&s_issued[cw]) = k + 1;
          }
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(&s_issued[CW - 1], 1);
        }
      } else if (lane == 0) {
        int published[kSenders];
#pragma unroll
        for (int w = 0; w < kSenders; ++w) published[w] = 0;
        const long long start = clock64();
        for (;;) {
          const int done = *reinterpret_cast<volatile int*>(&s_issued[CW - 1]);
          int snap[kSenders];
          bool any = false;
#pragma unroll
          for (int w = 0; w < kSenders; ++w) {
            snap[w] = *reinterpret_cast<volatile int*>(&s_issued[w]);
            any = any || snap[w] > published[w];
          }
          if (!any) {
            if (done == kSenders || *abort_flag != 0) break;
            if (clock64() - start > p.wait_cycles + tc::kWaitCycles) break;   // senders set the error
            __nanosleep(200);
            continue;
          }
          // acquire (the hand-overs read above) + release (the flags below) in one fence;
          // its cumulativity extends to the senders' stores
          __threadfence_system();
#pragma unroll
          for (int w = 0; w < kSenders; ++w) {
            for (int k = published[w]; k < snap[w]; ++k) {
              const int u = (k * kSenders + w) * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
              const int b = u / slices, sl = u - b * slices;
              const int idx = (p.rank * blocks_per_owner + b) * kSliceFlagStride + sl;
              SLAPO_DBG_CHECK(idx >= 0 && idx < 2 * kChunkCountOffset, p.status)
              for (int r = 0; r < p.world; ++r)
                *reinterpret_cast<volatile int*>(p.peer_chunk_flags[r] + idx) = p.epoch;
            }
            published[w] = snap[w];
          }
        }
        trace_mark(p.trace, 2);     // every slice of this CTA is published
      }
    } else if (staged && p.world > 1) {
      const int ct = threadIdx.x - 192;
      // A 128-row block is copied as `slices` slices by (usually) different CTAs, units in
      // (block, slice) order, so that the first blocks are complete after a few NVLink round
      // trips instead of all blocks becoming visible at the same late moment.
      const int slices = p.ag_slices;
      const int slice_rows = CBM / slices;
      int* chunk_count = p.chunk_flags + kChunkCountOffset;
      const int64_t slice_vec = static_cast<int64_t>(slice_rows) * p.row_bytes / 16;
      int u = 0;
      bool ok = true, marked = false;
      uint32_t owner_seen = 0;    // owners whose "entered" flag this CTA has observed
      // units in (block, owner, slice) order: at any moment the CTAs of this GPU pull from
      // all peers at once, and block b of every owner is complete before block b + 1
      for (int b = 0; b < blocks_per_owner && ok; ++b) {
        for (int o_idx = 1; o_idx < p.world && ok; ++o_idx) {
          const int owner = (p.rank + o_idx) % p.world;
          for (int sl = 0; sl < slices; ++sl, ++u) {
            if (u % static_cast<int>(gridDim.x) != static_cast<int>(blockIdx.x)) continue;
            if (!(owner_seen & (1u << owner))) {
              int w = 1;
              if (ct == 0) w = wait_flag(ready + owner, p.epoch, p.wait_cycles, abort_flag) ? 1 : 0;
              w = __syncthreads_or_named<CW * 32>(w);
              if (!w) { ok = false; break; }
              owner_seen |= 1u << owner;
            }
            const int64_t off = (static_cast<int64_t>(b) * CBM + sl * slice_rows) * p.row_bytes;
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const uint8_t*>(p.seg_src[owner]) + off);
            const int m_blk = owner * blocks_per_owner + b;
            SLAPO_DBG_CHECK(off + static_cast<int64_t>(slice_rows) * p.row_bytes <=
                                    static_cast<int64_t>(p.seg_len) * p.row_bytes &&
                                m_blk < kChunkCountOffset && (off & 15) == 0 &&
                                (static_cast<int64_t>(m_blk) * CBM + sl * slice_rows + slice_rows) <= p.M,
                            p.status)
            uint4* dst = reinterpret_cast<uint4*>(
                static_cast<uint8_t*>(p.stage_dst) +
                (static_cast<int64_t>(m_blk) * CBM + sl * slice_rows) * p.row_bytes);
            // 8 or 16 16-byte loads per thread are issued before the first store: with 128
            // threads that keeps 16 or 32 KB per SM on the wire to cover the NVLink round trip.
            if (ct == 0 && !marked) { trace_mark(p.trace, 1); marked = true; }
            if (p.ag_inflight == 16) copy_vecs<16, CW * 32>(src, dst, slice_vec, ct);
            else copy_vecs<8, CW * 32>(src, dst, slice_vec, ct);
            __threadfence();
            asm volatile("bar.sync 2, %0;" ::"n"(CW * 32) : "memory");
            if (ct == 0) {
              // the copier that completes the block publishes it
              const int prev = slices > 1 ? atomicAdd(chunk_count + m_blk, 1) : 0;
              if (prev + 1 == slices) {
                if (slices > 1) atomicExch(chunk_count + m_blk, 0);
                st_release_sys(p.chunk_flags + m_blk, p.epoch);
              }
            }
          }
        }
      }
      if (ct == 0) trace_mark(p.trace, 2);
    } else if (scatter) {
      // ------------------------------ reducer warps -------------------------------
      // Reduce-scatter / all-reduce: as soon as a 128-row block of this rank's rows is complete
      // in every rank's partial-product buffer (flags written by the epilogue warps of all
      // ranks), 32-row slices of it are pulled from all ranks over NVLink, summed in fp32,
      // finished with bias / activation and written out - while the main loop computes the
      // later blocks (see reduce_units).
      if constexpr (CW == 4) {
        trace_mark(threadIdx.x == 192 ? p.trace : 0, 1);
        reduce_units(p, rows_per_rank, blocks_per_owner, threadIdx.x - 192, 2, &s_red_next,
                     s_red_vote[0], abort_flag, &s_pipe_free, tc::smem_u32(smem));
        trace_mark(threadIdx.x == 192 ? p.trace : 0, 2);
        // all-reduce: the reduced rows stored to the peers must be visible before done2
        if (p.mode == kModeAllReduce) __threadfence_system();
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;
    int iter = 0;
    bool ok = true;
    uint32_t seen_ready = 1u << p.rank;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++iter) {
      int m_blk, n_blk;
      tile_coords(t, tiles_n, blocks_per_owner, p.world, p.rank, rotate, m_blk, n_blk, first,
                    scatter, staged);
      const int m0 = m_blk * CBM, n0 = n_blk * BN;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      int owner = p.rank;
      uint8_t* dst_base;
      int64_t dst_ld;
      int row_off = 0;
      if (scatter) {
        owner = m0 / rows_per_rank;
        // the partial tile stays in this rank's own symmetric buffer [M, N];
        // the owner of the rows pulls it with wide coalesced loads
        dst_base = static_cast<uint8_t*>(p.peer_recv[p.rank]);
        dst_ld = p.N;
        row_off = 0;
        if (!(seen_ready & (1u << owner))) {
          // the owner must have left its previous consumers of the buffer
          bool w = true;
          if (lane == 0) w = wait_flag(ready + owner, p.epoch, p.wait_cycles, abort_flag);
          w = __shfl_sync(0xffffffffu, w ? 1 : 0, 0) != 0;
          if (!w) { ok = false; break; }
          seen_ready |= 1u << owner;
        }
      } else {
        dst_base = static_cast<uint8_t*>(p.out);
        dst_ld = p.ldo;
      }
      if (!tc::mbar_wait_warp(&tmem_full[acc], acc_phase, abort_flag, mbar_budget)) { ok = false; break; }
      tc::fence_after_sync();
      const bool wide_store = dst_ld % 16 == 0 && (reinterpret_cast<uintptr_t>(dst_base) & 31) == 0;
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
            if (!scatter) {
              if (p.bias != nullptr) {
                const int cc = min(col0 + 2 * j, p.N - 2);
                v0 += cload(p.bias, cc, p.bf16);
                v1 += cload(p.bias, cc + 1, p.bf16);
              }
              if (p.act >= 0) {
                v0 = act_fwd(v0, p.act);
                v1 = act_fwd(v1, p.act);
              }
            }
            packed[j] = cpack2(v0, v1, p.bf16);
          }
          uint8_t* dst = dst_base + (static_cast<int64_t>(row - row_off) * dst_ld + col0) * 2;
          if (wide_store && col0 + 32 <= p.N) {
            // whole 32-byte sectors per store: a 16-byte store makes L2 merge two partial writes
#pragma unroll
            for (int v = 0; v < 2; ++v)
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(
                               dst + v * 32),
                           "r"(packed[8 * v]), "r"(packed[8 * v + 1]), "r"(packed[8 * v + 2]),
                           "r"(packed[8 * v + 3]), "r"(packed[8 * v + 4]), "r"(packed[8 * v + 5]),
                           "r"(packed[8 * v + 6]), "r"(packed[8 * v + 7])
                           : "memory");
          } else {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < p.N)
                *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(
                    packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
            }
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&tmem_empty[acc]);
      if (scatter) {
        // publish: make this warp's stores visible, count it; the warp that completes the row
        // block (all column tiles) raises the block's flag in THIS rank's buffer header.  The
        // owner polls that word over NVLink (see reduce_units), so the tensor-core pipeline
        // never waits for a store to a peer to be acknowledged.
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          const int prev = atomicAdd(p.blk_counters + m_blk, 1);
          if (prev + 1 == tiles_n * 4) {
            atomicExch(p.blk_counters + m_blk, 0);
            st_release_sys(p.blk_flags + m_blk, p.epoch);
          }
        }
      }
    }
    trace_mark(threadIdx.x == 64 ? p.trace : 0, 5);
    if (scatter) {
      // tiles stored: the four epilogue warps become a second reducing group (all four enter,
      // whatever their own `ok`: the group's leader looks at the CTA-wide abort flag)
      if constexpr (CW == 4) {
        // Every accumulator of this CTA has been read, so every MMA has completed and every
        // TMA load has landed: the operand pipeline's shared memory is free for the reduction
        // (96 KB per group).  Not after an error: loads may still be in flight then.
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (threadIdx.x == 64 && *abort_flag == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");
          s_pipe_free = 1;
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        reduce_units(p, rows_per_rank, blocks_per_owner, threadIdx.x - 64, 3, &s_red_next,
                     s_red_vote[1], abort_flag, &s_pipe_free, tc::smem_u32(smem) + 96 * 1024);
        if (p.mode == kModeAllReduce) __threadfence_system();
      }
    }
  }

  // ------------------------------ all-reduce closing -----------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (p.mode == kModeAllReduce && *abort_flag == 0) {
    // count CTAs, the last one tells every rank that this rank's reduced rows are in place;
    // the kernel leaves when every rank has said so
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int prev = atomicAdd(counters + 8, 1);
      if (prev + 1 == static_cast<int>(gridDim.x)) {
        atomicExch(counters + 8, 0);
        __threadfence_system();
        for (int r = 0; r < p.world; ++r) st_release_sys(p.peer_flags[r] + 16 + p.rank, p.epoch);
      }
      for (int r = 0; r < p.world; ++r)
        if (!wait_flag(done2 + r, p.epoch, p.wait_cycles, abort_flag)) break;
    }
    __syncthreads();
  }

  // ------------------------------ teardown ------------------------------------
  __syncthreads();
  trace_mark(threadIdx.x == 0 ? p.trace : 0, 6);
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 4);
  if (scatter && threadIdx.x == 0) {
    // the last CTA to leave clears the reduction-unit counter for the next launch
    const int prev = atomicAdd(p.flags + 41, 1);
    if (prev + 1 == static_cast<int>(gridDim.x)) {
      atomicExch(p.flags + 41, 0);
      atomicExch(p.flags + 40, 0);
    }
  }
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------ //
// All-gather by peer loads: dst[r * seg : (r + 1) * seg] = segment of rank r,
// read from rank r's symmetric buffer with 16-byte coalesced loads.  Same
// flag protocol as above (announce, then wait for a peer before reading it).
struct PeerGatherParams {
  const void* src[kMaxRanks];
  void* dst;
  int64_t seg_bytes;
  int world, rank, epoch;
  int* flags;
  int* peer_flags[kMaxRanks];
  int* status;
  long long wait_cycles;
};

__global__ void __launch_bounds__(256) peer_gather_kernel(const PeerGatherParams p) {
  __shared__ int s_abort;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_abort = 0;
    if (blockIdx.x == 0)
      for (int r = 0; r < p.world; ++r) st_release_sys(p.peer_flags[r] + p.rank, p.epoch);
  }
  __syncthreads();
  const int64_t n_vec = p.seg_bytes / 16;
  for (int i = 0; i < p.world; ++i) {
    const int r = (p.rank + i) % p.world;  // local segment first
    if (threadIdx.x == 0)
      s_ok = (r == p.rank) || wait_flag(p.flags + r, p.epoch, p.wait_cycles, &s_abort);
    __syncthreads();
    if (!s_ok) break;
    const uint4* src = static_cast<const uint4*>(p.src[r]);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.dst) + r * p.seg_bytes);
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec;
         v += static_cast<int64_t>(gridDim.x) * blockDim.x)
      dst[v] = src[v];
    __syncthreads();
  }
  if (threadIdx.x == 0 && s_abort != 0 && p.status != nullptr) atomicExch(p.status, 5);
}

int launch_peer_gather(void* const* src_ptrs, void* dst, int64_t seg_bytes, int world, int rank,
                       int epoch, int* flags, int* const* peer_flags, int* status,
                       double wait_seconds, cudaStream_t stream) {
  if (seg_bytes % 16 || world < 1 || world > kMaxRanks) return 1;
  PeerGatherParams p{};
  for (int r = 0; r < world; ++r) {
    p.src[r] = src_ptrs[r];
    p.peer_flags[r] = peer_flags != nullptr ? peer_flags[r] : flags;
  }
  p.dst = dst; p.seg_bytes = seg_bytes; p.world = world; p.rank = rank; p.epoch = epoch;
  p.flags = flags; p.status = status;
  p.wait_cycles = static_cast<long long>(wait_seconds * 1.9e9);
  count_launch();
  peer_gather_kernel<<<sm_count() * 2, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ------------------------------------------------------------------------ //
// All-gather by peer stores: every rank writes its own segment into the gathered buffer of ALL
// ranks at offset rank * seg - one multicast store per 16 bytes where the buffers have an
// NVSwitch address, one store per rank otherwise - and leaves when every rank's segment has
// landed in ITS buffer.  Stores need no answer, so the copy runs at the rate of the links
// (8 GPUs, 32 MB per rank: 377 us = 623 GB/s into every GPU) with a few thousand threads.
// Protocol (flag pad words: ready[r] = r, done[r] = 8 + r, CTA counter = 42):
//   1. announce `epoch` in ready[rank] on every rank; wait for all ranks' ready - nobody's
//      buffer is written before its owner has entered (its readers of the previous contents,
//      earlier kernels of its stream, are complete by then);
//   2. copy; every thread fences (system scope), the last CTA to finish raises done[rank] on
//      every rank;
//   3. wait until done[r] >= epoch for all r: the kernel's end means "gathered".
struct PushGatherParams {
  const void* src;
  void* mc_dst;                 // multicast address of the gathered buffers (or null)
  void* peer_dst[kMaxRanks];
  int64_t seg_bytes;
  int world, rank, epoch;
  int* flags;
  int* peer_flags[kMaxRanks];
  int* status;
  long long wait_cycles;
};

__global__ void __launch_bounds__(512) peer_push_gather_kernel(const PushGatherParams p) {
  __shared__ int s_abort;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_abort = 0;
    s_ok = 1;
    if (blockIdx.x == 0)
      for (int r = 0; r < p.world; ++r) st_release_sys(p.peer_flags[r] + p.rank, p.epoch);
  }
  __syncthreads();
  if (threadIdx.x < p.world && threadIdx.x != p.rank &&
      !wait_flag(p.flags + threadIdx.x, p.epoch, p.wait_cycles, &s_abort))
    s_ok = 0;
  __syncthreads();
  if (s_ok) {
    const int64_t n_vec = p.seg_bytes / 16;
    const uint4* src = static_cast<const uint4*>(p.src);
    const int64_t base = static_cast<int64_t>(p.rank) * p.seg_bytes;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; v + 3 * stride < n_vec; v += 4 * stride) {
      uint4 t[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) t[q] = __ldcg(src + v + q * stride);
      if (p.mc_dst != nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          mc_st(static_cast<uint8_t*>(p.mc_dst) + base + (v + q * stride) * 16, t[q]);
      } else {
        for (int rr = 0; rr < p.world; ++rr) {
          const int r = (p.rank + 1 + rr) % p.world;
          uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peer_dst[r]) + base);
#pragma unroll
          for (int q = 0; q < 4; ++q) d[v + q * stride] = t[q];
        }
      }
    }
    for (; v < n_vec; v += stride) {
      const uint4 t = __ldcg(src + v);
      if (p.mc_dst != nullptr) {
        mc_st(static_cast<uint8_t*>(p.mc_dst) + base + v * 16, t);
      } else {
        for (int r = 0; r < p.world; ++r)
          reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peer_dst[r]) + base)[v] = t;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA tells every rank that this rank's segment is in place
    const int prev = atomicAdd(p.flags + 42, 1);
    if (prev + 1 == static_cast<int>(gridDim.x)) {
      atomicExch(p.flags + 42, 0);
      __threadfence_system();
      if (s_abort == 0 && s_ok)
        for (int r = 0; r < p.world; ++r) st_release_sys(p.peer_flags[r] + 8 + p.rank, p.epoch);
    }
  }
  if (s_ok && threadIdx.x < p.world && !wait_flag(p.flags + 8 + threadIdx.x, p.epoch, p.wait_cycles, &s_abort))
    s_ok = 0;
  __syncthreads();
  if (threadIdx.x == 0 && (s_abort != 0 || s_ok == 0) && p.status != nullptr) atomicExch(p.status, 4);
}

int launch_peer_push_gather(const void* src, void* const* dst_ptrs, void* dst_mc, int64_t seg_bytes,
                            int world, int rank, int epoch, int* flags, int* const* peer_flags,
                            int* status, double wait_seconds, cudaStream_t stream) {
  if (seg_bytes % 16 || world < 1 || world > kMaxRanks || dst_ptrs == nullptr) return 1;
  PushGatherParams p{};
  for (int r = 0; r < world; ++r) {
    p.peer_dst[r] = dst_ptrs[r];
    p.peer_flags[r] = peer_flags != nullptr ? peer_flags[r] : flags;
  }
  p.src = src; p.mc_dst = world > 1 ? dst_mc : nullptr; p.seg_bytes = seg_bytes; p.world = world;
  p.rank = rank; p.epoch = epoch; p.flags = flags; p.status = status;
  p.wait_cycles = static_cast<long long>(wait_seconds * 1.9e9);
  count_launch();
  // one CTA per SM: every CTA waits for the peers at the end, so all of them must be resident
  peer_push_gather_kernel<<<sm_count(), 512, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ------------------------------------------------------------------------ //
template <int BN, int STAGES, bool A_MN, bool B_MN, int CW>
static int launch_comm_kernel(const SegMaps& ma, const SegMaps& mb, const CommGemmParams& p,
                              int grid, int threads, cudaStream_t stream) {
  using S = CommSmem<BN, STAGES>;
  auto kernel = comm_gemm_kernel<BN, STAGES, A_MN, B_MN, CW>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) !=
        cudaSuccess)
      return 3;
    configured = true;
  }
  count_launch();
  kernel<<<grid, threads, S::kTotal, stream>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_comm_variant(const SegMaps& ma, const SegMaps& mb, const CommGemmParams& p,
                               cudaStream_t stream) {
  const int tiles = ((p.M + CBM - 1) / CBM) * ((p.N + BN - 1) / BN);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.mode != kModeLocal) grid = sm_count();  // all CTAs take part in the reduction
  if constexpr (!A_MN) {
    // Staged gather (the launch checks rule out a transposed A here).  The variant with eight
    // copier warps (64 KB per SM in flight) measured slower than four warps at 2 and at 8 GPUs
    // (qkv / fc1 of BERT-large: 150 / 181 us against 140 / 159 us, 813 / 792 us against
    // 647 / 729 us); SLAPO_B200_AG_WIDE=1 selects it for experiments.
    static const bool wide = [] {
      const char* e = std::getenv("SLAPO_B200_AG_WIDE");
      return e != nullptr && e[0] == '1';
    }();
    if (p.gather == 4 && wide)
      return launch_comm_kernel<BN, STAGES, A_MN, B_MN, 8>(ma, mb, p, grid, 192 + 8 * 32, stream);
    if (p.gather == 4 || p.gather == 5)
      return launch_comm_kernel<BN, STAGES, A_MN, B_MN, 4>(ma, mb, p, grid, 320, stream);
  }
  // scatter modes: four reducer warps; otherwise the six warps of the plain pipeline
  return launch_comm_kernel<BN, STAGES, A_MN, B_MN, 4>(ma, mb, p, grid,
                                                       p.mode != kModeLocal ? 320 : 192, stream);
}

// Tuning of the staged gather's copier warps, read once from SLAPO_B200_AG_COPY="slices,inflight"
// (slices per 128-row block: 1, 2 or 4; 16-byte loads in flight per thread: 8 or 16).
struct CopyTuning { int slices, inflight; };
static CopyTuning copy_tuning() {
  static const CopyTuning t = [] {
    CopyTuning v{kDefaultAgSlices, kDefaultAgInflight};
    if (const char* e = std::getenv("SLAPO_B200_AG_COPY")) {
      int a = 0, b = 0;
      if (std::sscanf(e, "%d,%d", &a, &b) == 2 && (a == 1 || a == 2 || a == 4) && (b == 8 || b == 16)) {
        v.slices = a;
        v.inflight = b;
      }
    }
    return v;
  }();
  return t;
}

// The pushed gather's tuning, SLAPO_B200_AG_PUSH="slices,inflight": slices per 128-row block
// (1 .. 16, a power of two - one slice is one warp's unit of work) and 16-byte loads in flight
// per lane (8 or 16).
static CopyTuning push_tuning() {
  static const CopyTuning t = [] {
    CopyTuning v{16, 16};
    if (const char* e = std::getenv("SLAPO_B200_AG_PUSH")) {
      int a = 0, b = 0;
      if (std::sscanf(e, "%d,%d", &a, &b) == 2 && a >= 1 && a <= kSliceFlagStride && (a & (a - 1)) == 0 &&
          (b == 8 || b == 16)) {
        v.slices = a;
        v.inflight = b;
      }
    }
    return v;
  }();
  return t;
}

// Copies the phase trace of the last fused kernel ([kTraceCtas][kTraceSlots] 64-bit words) to the host.
int read_comm_trace(unsigned long long* host, int n_words) {
  const int n = n_words < kTraceCtas * kTraceSlots ? n_words : kTraceCtas * kTraceSlots;
  return cudaMemcpyFromSymbol(host, g_comm_trace, static_cast<size_t>(n) * 8) == cudaSuccess ? 0 : 1;
}

// a_ptrs / b_ptrs: one base pointer per segment (rank) when the operand is
// gathered, else only entry 0 is used.  Shapes follow gemm.cu (a_mn / b_mn).
int launch_comm_gemm(void* const* a_ptrs, void* const* b_ptrs, int M, int N, int K, int lda,
                     int ldb, bool a_mn, bool b_mn, bool bf16, int gather, int seg_len, int mode,
                     int world, int rank, int epoch, void* out, int ldo, const void* bias, int act,
                     int* flags, int* const* peer_flags, void* const* peer_recv,
                     void* const* peer_out, int* status, double wait_seconds, void* stage_dst,
                     int* chunk_flags, void* recv_mc, void* out_mc, void* const* stage_peers,
                     void* stage_mc, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((gather == 4 || gather == 5 || mode != kModeLocal) && (M + CBM - 1) / CBM > kChunkCountOffset)
    return 6;
  if ((gather == 4 || gather == 5) && mode != kModeLocal) return 1;   // warps 6-9 have one job per launch
  if (gather == 5) {
    // pushed gather: every rank's staging slot = kRecvHeaderBytes of block flags and slice
    // counters (zero when allocated, flags only grow), then the gathered operand [M, K]
    if (a_mn || stage_peers == nullptr || lda != K || seg_len % CBM != 0 || seg_len * world != M)
      return 1;
    // the header holds kSliceFlagStride flag words per 128-row block
    if ((M / CBM) * kSliceFlagStride > 2 * kChunkCountOffset) return 6;
    for (int r = 0; r < world; ++r)
      if (stage_peers[r] == nullptr || (reinterpret_cast<uintptr_t>(stage_peers[r]) & 15)) return 1;
    stage_dst = static_cast<uint8_t*>(stage_peers[rank]) + kRecvHeaderBytes;
    chunk_flags = reinterpret_cast<int*>(stage_peers[rank]);
  }
  if (mode != kModeLocal && peer_recv == nullptr) return 1;
  if (gather == 4 && (a_mn || stage_dst == nullptr || chunk_flags == nullptr || lda != K ||
                      seg_len % CBM != 0 || seg_len * world != M))
    return 1;
  if (N % 8 || K % 8 || lda % 8 || ldb % 8 || ldo % 8) return 1;
  if (world < 1 || world > kMaxRanks) return 1;
  if (a_mn && M % 8) return 1;
  if (mode != kModeLocal && (M % world != 0 || (M / world) % CBM != 0)) return 1;
  if (gather == 1 && (seg_len % CBM != 0 || seg_len * world != M)) return 1;
  if ((gather == 2 || gather == 3) && (seg_len % CBK != 0 || seg_len * world != K)) return 1;
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  SegMaps ma, mb;
  const int a_segs = (gather == 1 || gather == 2) ? world : 1;
  const int b_segs = gather == 3 ? world : 1;
  if (gather == 4 || gather == 5) {
    // map 0: this rank's shard in place; map 1: the local staging buffer [M, K]
    if (!make_tmap_2d(&ma.map[0], a_ptrs[rank], K, seg_len, lda, 64, CBM, 2, bf16) ||
        !make_tmap_2d(&ma.map[1], stage_dst, K, M, lda, 64, CBM, 2, bf16))
      return 2;
  }
  for (int s = 0; s < a_segs && gather != 4 && gather != 5; ++s) {
    // extents of one segment
    const uint64_t rows = gather == 1 ? seg_len : M;
    const uint64_t kk = gather == 2 ? seg_len : K;
    const bool ok = a_mn ? make_tmap_2d(&ma.map[s], a_ptrs[s], rows, kk, lda, 64, CBK, 2, bf16)
                         : make_tmap_2d(&ma.map[s], a_ptrs[s], kk, rows, lda, 64, CBM, 2, bf16);
    if (!ok) return 2;
  }
  for (int s = 0; s < b_segs; ++s) {
    const uint64_t kk = gather == 3 ? seg_len : K;
    const bool ok = b_mn ? make_tmap_2d(&mb.map[s], b_ptrs[s], N, kk, ldb, 64, CBK, 2, bf16)
                         : make_tmap_2d(&mb.map[s], b_ptrs[s], kk, N, ldb, 64, BN, 2, bf16);
    if (!ok) return 2;
  }
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.world = world; p.rank = rank; p.gather = gather;
  p.seg_len = seg_len > 0 ? seg_len : 1; p.mode = mode; p.epoch = epoch; p.out = out; p.ldo = ldo;
  p.bias = bias; p.act = act; p.bf16 = bf16 ? 1 : 0; p.flags = flags; p.status = status;
  p.idesc = tc::instr_desc_f16(CBM, BN, bf16 ? 1 : 0, a_mn, b_mn);
  p.wait_cycles = static_cast<long long>(wait_seconds * 1.9e9);
  p.stage_dst = stage_dst; p.chunk_flags = chunk_flags; p.row_bytes = K * 2;
  const CopyTuning tune = gather == 5 ? push_tuning() : copy_tuning();
  p.ag_slices = tune.slices; p.ag_inflight = tune.inflight;
  // a slice is whole rows of 16-byte vectors
  if (gather == 5 && (K * 2) % 16 != 0) return 1;
  static const bool trace_on = [] {
    const char* e = std::getenv("SLAPO_B200_COMM_TRACE");
    return e != nullptr && e[0] == '1';
  }();
  p.trace = trace_on ? 1 : 0;
  for (int r = 0; r < world; ++r) {
    p.seg_src[r] = gather == 4 || (gather == 5 && r == rank) ? a_ptrs[r] : nullptr;
    if (gather == 5) {
      p.peer_chunk_flags[r] = reinterpret_cast<int*>(stage_peers[r]);
      p.peer_stage[r] = static_cast<uint8_t*>(stage_peers[r]) + kRecvHeaderBytes;
    }
    p.peer_flags[r] = peer_flags != nullptr ? peer_flags[r] : flags;
    // a partial-product buffer starts with kRecvHeaderBytes of block flags (written by the
    // peers) and arrival counters (local), zero when the buffer was allocated
    uint8_t* recv = peer_recv != nullptr ? static_cast<uint8_t*>(peer_recv[r]) : nullptr;
    p.peer_blk_flags[r] = reinterpret_cast<int*>(recv);
    p.peer_recv[r] = recv != nullptr ? recv + kRecvHeaderBytes : nullptr;
    p.peer_out[r] = peer_out != nullptr ? peer_out[r] : nullptr;
  }
  if (recv_mc != nullptr && mode != kModeLocal && world > 1) {
    p.mc_blk_flags = reinterpret_cast<int*>(recv_mc);
    p.mc_recv = static_cast<uint8_t*>(recv_mc) + kRecvHeaderBytes;
    p.mc_out = mode == kModeAllReduce ? out_mc : nullptr;
  }
  if (gather == 5 && stage_mc != nullptr && world > 1)
    p.mc_stage = static_cast<uint8_t*>(stage_mc) + kRecvHeaderBytes;
  p.blk_flags = p.peer_blk_flags[rank];
  p.blk_counters = p.blk_flags != nullptr ? p.blk_flags + kChunkCountOffset : nullptr;

#define COMM_CASE(BN_, ST_)                                                                   \
  if (BN == BN_) {                                                                            \
    if (!a_mn && !b_mn) return launch_comm_variant<BN_, ST_, false, false>(ma, mb, p, stream); \
    if (!a_mn && b_mn) return launch_comm_variant<BN_, ST_, false, true>(ma, mb, p, stream);   \
    if (a_mn && !b_mn) return launch_comm_variant<BN_, ST_, true, false>(ma, mb, p, stream);   \
    return launch_comm_variant<BN_, ST_, true, true>(ma, mb, p, stream);                       \
  }
  COMM_CASE(256, 4)
  COMM_CASE(128, 6)
  COMM_CASE(64, 8)
#undef COMM_CASE
  return 1;
}

}  // namespace slapo
