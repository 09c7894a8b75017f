// Device-side pieces shared by the backward kernels (csrc/bwd_sm100.cu: preprocess, dQ kernel, dK/dV kernel;
// csrc/bwd_fused_sm100.cu: the single-kernel backward): kernel parameters, tile descriptors, the MMA issue
// helpers, and the hand-off helpers of the elementwise warps.
#pragma once

#include "common.h"

// The backward kernels keep the wait loops inline: with 96 registers per thread a call inside their loops costs
// spills around every wait (measured: dK/dV kernel 25 % slower at head size 128 with the out-of-line form).
#define FA_WAIT_INLINE
#define FA_WAIT_SLIM
#include "ptx.cuh"

namespace fa {

struct BwdKernelParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  __half* dq;
  __half* dk;
  __half* dv;
  int64_t dq_batch_stride, dq_row_stride, dq_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  const float* delta;  // (b, h, sq_pad), holds -rowsum(dO*O)
  const float* lse2;   // (b, h, sq_pad), holds -LSE*log2(e)
  int sq_pad;
  int seqlen_q, seqlen_k, h, h_k;
  float scale, scale_log2;
  int is_causal;
  int causal_shift;  // is_causal == 2: key j visible to query i iff j <= i + causal_shift (else sk - sq is used)
  const int* cu_seqlens_q;
  const int* cu_seqlens_k;
  int* status;
  // single-kernel backward: fp32 dQ accumulator (heads, dq_acc_rows, d), rows grouped in 128-row tiles;
  // the tiles of sequence b start at row dq_acc_tile_base(b) * 128
  float* dq_acc;
  int64_t dq_acc_rows;  // rows per head
  int total_q;
  // persistent dQ kernel: work counter pair (see next_sched_slot) and the extents of the index space
  int* sched;
  int items_x;      // dense: 128-row Q tiles per (sequence, head)
  int total_items;  // dense: items_x * h * b; packed sequences: h * (total_q / 128 + b)
  int b;
};

// Launchers of the single-kernel backward (bwd_fused_sm100.cu), called from fa_bwd_stages().
int launch_bwd_fused(const BwdKernelParams& kp, const FaBwdParams* p, cudaStream_t stream);
int launch_bwd_dq_finalize(const BwdKernelParams& kp, const FaBwdParams* p, cudaStream_t stream);

namespace {

constexpr int kBlock = 128;  // tile edge in both sequence dimensions
constexpr int kNumThreads = 608;  // 16 elementwise warps, TMA producer, two MMA-issuing warps
// 19 warps: five on one SM sub-partition (16384 registers) -> at most 96 registers per thread, which is what
// __launch_bounds__(608, 1) makes the compiler use; a larger budget could not be scheduled at all
static_assert((kNumThreads / 32 + 3) / 4 * 32 * 96 <= 16384, "register file of one SM sub-partition");
constexpr int kComputeWarps = 16;
constexpr int kProducerWarp = 16;
constexpr int kMmaWarp = 17;    // issues the products S, dP (S^T, dP^T) that feed the elementwise warps
constexpr int kAccMmaWarp = 18; // issues the accumulating products dQ (dV, dK)
constexpr int kTmemCols = 512;
constexpr int kColS = 0;
constexpr int kColDP = 128;
constexpr int kColAcc = 256;
constexpr int kColPacked = 384;  // dQ kernel: packed dS, two buffers of 64 columns
// dK/dV kernel: columns of dP^T.  At D = 128 the accumulators fill columns 256-511 and dP^T has to share
// region A with S^T; at D = 64 columns 384-511 are free, dP^T gets a region of its own and S^T(it+1) need
// not wait until dP^T(it) has been read.
template <int D>
constexpr int kColDPT = (D == 64) ? 384 : kColS;
__device__ __forceinline__ float2 exp2_pair(float2 x) { return make_float2(ex2f(x.x), ex2f(x.y)); }


// First accumulator tile of sequence `batch`: dense batches use the padded length, packed batches the tile
// that holds the sequence's first row plus one tile per preceding sequence (so that no two sequences share
// a tile and the total stays below total_q / 128 + batch count).
__device__ __forceinline__ int64_t dq_acc_tile_base(const BwdKernelParams& p, int batch, int q_off) {
  return p.cu_seqlens_q ? static_cast<int64_t>(q_off / 128 + batch) : static_cast<int64_t>(batch) * (p.sq_pad / 128);
}

template <int D>
struct BCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = (D == 128) ? 2 : 3;
  // dQ kernel: a K tile lives from the S MMAs of its block to the dQ MMAs one block later, a V tile only
  // for the dP MMAs, so K gets one stage more (3 x 32 KB + 2 x 32 KB + Q + dO = 224 KB at D = 128).
  static constexpr int kStagesK = kStages + 1;
  static constexpr int kStagesV = kStages;
  static constexpr int kSmemBytesDq = 2 * kTileBytes + (kStagesK + kStagesV) * kTileBytes + 512 /*barriers*/ +
                                      1024 /*alignment*/;
  // dK/dV kernel: a Q tile lives from the S^T MMAs of its iteration to the dK MMAs issued one iteration
  // later, a dO tile for less than one iteration; the row statistics have a ring of their own (2 x 1 KB)
  // that the elementwise warps release.  At D = 128 the tiles take 224 KB, which leaves no room for an
  // alignment pad: the kernel checks that the dynamic shared memory starts on a 1024-byte boundary.
  static constexpr int kStagesQ = kStages + 1;
  static constexpr int kStagesDO = kStages;
  static constexpr int kAlignPadDkdv = (D == 128) ? 0 : 1024;
  static constexpr int kSmemBytesDkdv = 2 * kTileBytes + (kStagesQ + kStagesDO) * kTileBytes + 2048 /*stats*/ +
                                        512 /*barriers*/ + kAlignPadDkdv;
  static_assert(kSmemBytesDq <= 227 * 1024 && kSmemBytesDkdv <= 227 * 1024, "shared memory budget");
};

struct BBarriers {
  uint64_t fixed_full;     // the tiles loaded once (Q,dO or K,V)
  uint64_t a_full[4];      // ring A (dQ: K, dK/dV: Q + stats)
  uint64_t a_empty[4];
  uint64_t b_full[4];      // ring B (dQ: V, dK/dV: dO)
  uint64_t b_empty[4];
  uint64_t s_full;         // S (or S^T) accumulator ready
  uint64_t dp_full;        // dP (or dP^T) accumulator ready
  uint64_t p_full;         // packed P^T written to TMEM (dK/dV kernel)
  uint64_t ds_full;        // packed dS (or dS^T) written to TMEM
  uint64_t s_loaded;       // S (S^T) sits in registers: its TMEM region may be overwritten
  uint64_t dp_loaded;      // dP (dP^T) sits in registers
  uint64_t p_free;         // dV MMAs of the previous tile have consumed the packed P^T
  uint64_t ds_free[2];     // dK/dV kernel [0]: dK MMAs of the previous tile have consumed the packed dS^T;
                           // dQ kernel [u]: the dQ MMAs have consumed packed-dS buffer u
  uint64_t st_full[2];     // dK/dV kernel: row statistics (lse, delta) of a Q tile loaded
  uint64_t st_empty[2];    // ... and read by all elementwise warps
  uint64_t tail_fixed[4];  // rows past the end of a packed sequence have been zeroed in an operand tile
                           // (dK/dV kernel: one barrier per dO stage -- up to 3 at head size 64 -- so that
                           // the producer cannot run two phases ahead of the waiting thread)
  uint64_t acc_full;       // final accumulators ready
  uint32_t tmem_base;
  int abort_flag;
};

// a_users / b_users: how many MMA-issuing threads read the tiles of ring A / B (each commits on "empty").
__device__ __forceinline__ void init_barriers(BBarriers* bars, int stages, int a_users, int b_users) {
  mbar_init(&bars->fixed_full, 1);
  for (int s = 0; s < stages; ++s) {
    mbar_init(&bars->a_full[s], 1);
    mbar_init(&bars->a_empty[s], a_users);
    mbar_init(&bars->b_full[s], 1);
    mbar_init(&bars->b_empty[s], b_users);
  }
  mbar_init(&bars->s_full, 1);
  mbar_init(&bars->dp_full, 1);
  mbar_init(&bars->p_full, kComputeWarps);
  mbar_init(&bars->ds_full, kComputeWarps);
  mbar_init(&bars->s_loaded, kComputeWarps);
  mbar_init(&bars->dp_loaded, kComputeWarps);
  for (int i = 0; i < 2; ++i) {
    mbar_init(&bars->st_full[i], 1);
    mbar_init(&bars->st_empty[i], kComputeWarps);
  }
  mbar_init(&bars->p_free, 1);
  mbar_init(&bars->ds_free[0], 1);
  mbar_init(&bars->ds_free[1], 1);
  for (int i = 0; i < 4; ++i) mbar_init(&bars->tail_fixed[i], 1);
  mbar_init(&bars->acc_full, 1);
  bars->abort_flag = 0;
  fence_mbar_init();
}

// Tile descriptors (built once per tile by the MMA thread) and their K=16 slices.
// K-major 128-row tile: slice k lives in swizzle chunk k/4 at byte (k%4)*32 inside the 128-byte row.
// MN-major use of the same tile (N = D): slice k is 16 rows (2048 B) further.
template <int D>
__device__ __forceinline__ uint64_t kmajor_tile(uint32_t tile_addr) { return make_smem_desc(tile_addr, 16, 1024); }
template <int D>
__device__ __forceinline__ uint64_t mnmajor_tile(uint32_t tile_addr) {
  return make_smem_desc(tile_addr, BCfg<D>::kChunkBytes, 1024);
}
template <int D>
__device__ __forceinline__ uint64_t kmajor_slice(uint64_t tile_desc, int k) {
  return desc_advance(tile_desc, (k >> 2) * BCfg<D>::kChunkBytes + (k & 3) * 32);
}
__device__ __forceinline__ uint64_t mnmajor_slice(uint64_t tile_desc, int k) { return desc_advance(tile_desc, k * 2048); }

// A thread that issues tcgen05.mma is held for the duration of each MMA (about 66 clocks for
// 128x128x16), and whatever else it executes -- a barrier poll costs 60-80 clocks even when the barrier
// completed long ago, a commit about 50 -- is time in which it feeds nothing to the tensor pipe.  Two
// measures keep the pipe busy: the products are issued by two warps (kMmaWarp, kAccMmaWarp), so that one
// polls while the other issues, and a product takes a hook that runs after half of its MMAs for waits on
// TMA loads of the NEXT product, which are satisfied long before and cost only the poll.  A hook returns
// false when a bounded wait gave up; the rest of the product is then skipped.
// C = A[smem, K-major] * B[smem, K-major]^T over D, both 128-row tiles.
template <int D, class Hook>
__device__ __forceinline__ bool gemm_ss(uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile, uint32_t idesc,
                                        Hook hook) {
  const uint64_t ad = kmajor_tile<D>(a_tile), bd = kmajor_tile<D>(b_tile);
  constexpr int kSlices = D / 16;
#pragma unroll
  for (int k = 0; k < kSlices; ++k) {
    if (k == kSlices / 2 && !hook()) return false;
    mma_ss(d_tmem, kmajor_slice<D>(ad, k), kmajor_slice<D>(bd, k), idesc, k > 0);
  }
  return true;
}
// C (+)= A[tmem, 128 packed fp16 contraction elements in 64 consecutive columns] * B[smem tile used
// MN-major, N = D].
template <int D>
__device__ __forceinline__ void gemm_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_tile, uint32_t idesc,
                                        bool zero_init) {
  const uint64_t bd = mnmajor_tile<D>(b_tile);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    mma_ts(d_tmem, a_tmem + k * 8, mnmajor_slice(bd, k), idesc, (zero_init && k == 0) ? 0u : 1u);
}

// Rows of a packed (varlen) tensor past the end of a sequence belong to the NEXT sequence.  Their scores are
// masked (P = 0, dS = 0 by selection), but as operand rows of an accumulating MMA they would still be
// multiplied by those zeros, and 0 x NaN/Inf in a neighbour's data would poison this sequence's gradients.
// Whole 128-byte row segments of the swizzled tile are zeroed (the swizzle only permutes 16-byte units
// inside a row); executed by all lanes of one warp, visible to the tensor core after the fence.
template <int D>
__device__ __forceinline__ void zero_tile_rows_from(uint8_t* tile, int first_row, int lane) {
  using C = BCfg<D>;
  for (int idx = lane; idx < (kBlock - first_row) * C::kChunks * 8; idx += 32) {
    const int r = first_row + idx / (C::kChunks * 8);
    const int u = idx % (C::kChunks * 8);
    *reinterpret_cast<uint4*>(tile + (u >> 3) * C::kChunkBytes + r * 128 + (u & 7) * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  __syncwarp();
}

// One warp's arrival on a barrier that counts warps: all lanes have finished their TMEM stores.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  tmem_wait_st();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
// A poll of a barrier costs the elementwise warps 100-170 clocks even when it completed long ago, so the
// barriers that normally complete early are probed ahead of time, with independent work (a TMEM load,
// the arithmetic of a phase) between the probe and its use; the blocking wait runs only if the probe
// failed.  The vote makes the result uniform over the warp.
__device__ __forceinline__ bool warp_probe(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_test_nonblocking(bar, parity) != 0);
}
__device__ __forceinline__ bool warp_wait_unless(bool probed, uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  return probed || mbar_wait_warp(bar, parity, ctx);
}
// The same after TMEM loads (tcgen05.wait::ld already executed): the region may be overwritten.
__device__ __forceinline__ void warp_arrive_loaded(uint64_t* bar, int lane) {
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

__device__ __forceinline__ void store_row_fp16(__half* dst, const uint32_t (&r)[32], float mul) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack_half2(__uint_as_float(r[8 * i + 0]) * mul, __uint_as_float(r[8 * i + 1]) * mul);
    v.y = pack_half2(__uint_as_float(r[8 * i + 2]) * mul, __uint_as_float(r[8 * i + 3]) * mul);
    v.z = pack_half2(__uint_as_float(r[8 * i + 4]) * mul, __uint_as_float(r[8 * i + 5]) * mul);
    v.w = pack_half2(__uint_as_float(r[8 * i + 6]) * mul, __uint_as_float(r[8 * i + 7]) * mul);
    *reinterpret_cast<uint4*>(dst + i * 8) = v;
  }
}

}  // namespace
}  // namespace fa
