// Backward attention for sm_100a: dQ, dK, dV from dO, O and LSE.  Three kernels on one stream:
//
//   1. preprocess   -delta[b,h,i] = -sum_d dO*O (fp32) and -lse2 = -LSE*log2(e) (stored negated so that
//                   the consumers need only fused multiply-adds), both padded to a multiple of 128 rows
//                   per (b, h); padded rows get -lse2 = -inf so that they produce P = 0.
//   2. dQ kernel    one CTA per 128-row Q tile; loops over K/V blocks:
//                     S  = Q K_j^T, dP = dO V_j^T            (tcgen05 SS, fp32 in TMEM)
//                     P  = exp2(S*c - lse2), dS = P o (dP - delta) -> fp16, written to TMEM columns of its own
//                     dQ += dS K_j                            (tcgen05 TS, K_j as MN-major B operand)
//   3. dK/dV kernel one CTA per 128-key tile of one KV head; loops over the query heads of the GQA
//                   group and their Q tiles, accumulating in TMEM (fp32) so that dK/dV are written
//                   once per KV head:
//                     S^T = K Q_i^T, dP^T = V dO_i^T          (SS)
//                     P^T, dS^T -> fp16 in TMEM columns of their own
//                     dV += P^T dO_i, dK += dS^T Q_i          (TS, dO_i / Q_i as MN-major B operands)
// Warp roles in kernels 2 and 3 (608 threads): warps 0-15 elementwise math (four threads per TMEM lane,
// each owning 32 of the 128 columns of a tile), warp 16 TMA producer, warp 17 issues the SS products
// that feed the elementwise warps, warp 18 the accumulating TS products.
// TMEM columns.  dQ kernel: S [0,128), dP [128,256), dQ [256,256+D), packed dS double-buffered in
// [384,448) / [448,512).  dK/dV kernel: one 128-column accumulator region A [0,128) that holds S^T and
// then dP^T of the same Q tile in turn, packed P^T [128,192) and dS^T [192,256), dV [256,256+D),
// dK [256+D,256+2D) (at D = 64 columns 384-511 are left over and dP^T gets them as a region of its own).
// A region is handed back to the MMA warp as soon as its values sit in registers, so the next S / dP /
// S^T is computed while the elementwise warps are still busy with the current tile.
//
// Replaces flash_bwd_dot_do_o_kernel (csrc/flash_attn/src/flash_bwd_preprocess_kernel.h:23-96),
// compute_dq_1rowblock and compute_dk_dv_1colblock (src/flash_bwd_kernel.h:25-609, 613-1344) and
// the GQA group sum torch::sum_out (csrc/flash_attn/flash_api.cpp:338-348) of the reference.
#include "common.h"
#include "ptx.cuh"

namespace fa {
namespace {

constexpr int kBlock = 128;  // tile edge in both sequence dimensions
constexpr int kNumThreads = 608;  // 16 elementwise warps, TMA producer, two MMA-issuing warps
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
  const int* cu_seqlens_q;
  const int* cu_seqlens_k;
  int* status;
};

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

// =============================================================================================
// 1. preprocess
// =============================================================================================
struct PreParams {
  const __half* o;
  const __half* dout;
  const float* lse;
  float* delta;
  float* lse2;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  int64_t lse_row_stride;
  int h, seqlen_q, sq_pad, d;
  const int* cu_seqlens_q;
};

// Work item = (group of kPreRows consecutive rows, head), heads fastest, d/8 threads per item (16-byte loads):
// the threads of a block read neighbouring heads of the same rows, i.e. contiguous memory when the heads of a
// row are adjacent, every thread has 2 * kPreRows loads in flight, and an item writes one full 32-byte sector
// of each statistic.  grid (ceil(items / items_per_block), 1, b).
constexpr int kPreRows = 8;
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const PreParams p) {
  const int tpr = p.d / 8;  // threads per item: 8 or 16
  const int item = blockIdx.x * (256 / tpr) + threadIdx.x / tpr;
  const int sub = threadIdx.x % tpr;
  const int head = item % p.h, row0 = (item / p.h) * kPreRows;
  const int batch = blockIdx.z;
  // items past the end take part in the shuffles and touch no memory (every access below is bounded)
  const int q_off = p.cu_seqlens_q ? p.cu_seqlens_q[batch] : 0;
  const int sq = p.cu_seqlens_q ? p.cu_seqlens_q[batch + 1] - q_off : p.seqlen_q;
  const int64_t o_base = (p.cu_seqlens_q ? static_cast<int64_t>(q_off) * p.o_row_stride : batch * p.o_batch_stride) +
                         head * p.o_head_stride + sub * 8;
  const int64_t do_base = (p.cu_seqlens_q ? static_cast<int64_t>(q_off) * p.do_row_stride : batch * p.do_batch_stride) +
                          head * p.do_head_stride + sub * 8;
  uint4 a[kPreRows], b[kPreRows];
#pragma unroll
  for (int i = 0; i < kPreRows; ++i) {
    a[i] = make_uint4(0, 0, 0, 0);
    b[i] = make_uint4(0, 0, 0, 0);
    if (row0 + i < sq) {
      a[i] = *reinterpret_cast<const uint4*>(p.o + o_base + static_cast<int64_t>(row0 + i) * p.o_row_stride);
      b[i] = *reinterpret_cast<const uint4*>(p.dout + do_base + static_cast<int64_t>(row0 + i) * p.do_row_stride);
    }
  }
  // lane `sub` of the item keeps the statistics of row `sub` (sub < kPreRows <= tpr)
  const int64_t bh = static_cast<int64_t>(batch) * p.h + head;
  float my_lse = 0.f;
  if (sub < kPreRows && row0 + sub < sq) my_lse = p.lse[bh * p.lse_row_stride + row0 + sub];
  float mine = 0.f;
#pragma unroll
  for (int i = 0; i < kPreRows; ++i) {
    const __half2* ah = reinterpret_cast<const __half2*>(&a[i]);
    const __half2* bh2 = reinterpret_cast<const __half2*>(&b[i]);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __half22float2(ah[k]), y = __half22float2(bh2[k]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
    // sum over the tpr (8 or 16) consecutive lanes of the item; every lane ends up with the total
    for (int off = tpr / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == i) mine = acc;
  }
  if (sub < kPreRows && row0 + sub < p.sq_pad) {
    const int64_t idx = bh * p.sq_pad + row0 + sub;
    const bool valid = row0 + sub < sq;
    p.delta[idx] = valid ? -mine : 0.f;
    p.lse2[idx] = valid ? -my_lse * kLog2e : -INFINITY;
  }
}

// =============================================================================================
// 2. dQ kernel
// =============================================================================================
template <int D>
__global__ void __launch_bounds__(kNumThreads, 1)
bwd_dq_kernel(const __grid_constant__ BwdKernelParams p) {
  using C = BCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const int batch = blockIdx.z, head = blockIdx.y;
  const int mblk = gridDim.x - 1 - blockIdx.x;
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int q_off = varlen ? p.cu_seqlens_q[batch] : 0;
  const int sq = varlen ? p.cu_seqlens_q[batch + 1] - q_off : p.seqlen_q;
  const int k_off = varlen ? p.cu_seqlens_k[batch] : 0;
  const int sk = varlen ? p.cu_seqlens_k[batch + 1] - k_off : p.seqlen_k;
  const int row0 = mblk * kBlock;
  if (row0 >= sq) return;
  if (p.status && (*reinterpret_cast<volatile int*>(p.status) & kStatusWaitTimeout) != 0) return;
  const int bq = varlen ? 0 : batch;
  const int head_k = head / (p.h / p.h_k);
  const int nkb = (sk + kBlock - 1) / kBlock;
  int nb = nkb;
  if (p.is_causal) {
    const int x = row0 + kBlock + sk - sq;
    nb = x <= 0 ? 0 : min(nkb, (x + kBlock - 1) / kBlock);
  }

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::kTileBytes;
  uint8_t* sK = sdO + C::kTileBytes;
  uint8_t* sV = sK + C::kStagesK * C::kTileBytes;
  BBarriers* bars = reinterpret_cast<BBarriers*>(sV + C::kStagesV * C::kTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The TMA producer thread initialises the barriers itself and issues the loads of Q, dO and of the first
  // K/V blocks BEFORE the CTA-wide synchronisation, so that their latency overlaps the TMEM allocation.
  WaitCtx ctx{&bars->abort_flag, p.status};
  auto load_kv = [&](int j) -> bool {
    const int s = j % C::kStagesK, sv = j % C::kStagesV;
    const uint32_t ph = (j / C::kStagesK) & 1, phv = (j / C::kStagesV) & 1;
    const int krow = k_off + j * kBlock;
    if (!mbar_wait(&bars->a_empty[s], ph ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->a_full[s], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sK + s * C::kTileBytes + c * C::kChunkBytes, &p.tm_k, &bars->a_full[s], c * 64, head_k, krow, bq);
    if (!mbar_wait(&bars->b_empty[sv], phv ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->b_full[sv], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sV + sv * C::kTileBytes + c * C::kChunkBytes, &p.tm_v, &bars->b_full[sv], c * 64, head_k, krow, bq);
    return true;
  };
  const int n_early = min(nb, C::kStagesV);  // stages that are free from the start: no wait blocks
  if (warp == kProducerWarp && lane == 0) {
    init_barriers(bars, C::kStagesK, 2, 1);
    if (nb > 0) {
      mbar_arrive_expect_tx(&bars->fixed_full, 2 * C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(sQ + c * C::kChunkBytes, &p.tm_q, &bars->fixed_full, c * 64, head, q_off + row0, bq);
        tma_load_4d(sdO + c * C::kChunkBytes, &p.tm_do, &bars->fixed_full, c * 64, head, q_off + row0, bq);
      }
      for (int j = 0; j < n_early; ++j) load_kv(j);
    }
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  // the last K block of a packed sequence holds rows of the next sequence (see zero_tile_rows_from)
  const bool fix_k_tail = varlen && (sk % kBlock) != 0 && nb == nkb && nb > 0;
  if (warp == kProducerWarp) {
    if (lane == 0) {
      for (int j = n_early; j < nb; ++j)
        if (!load_kv(j)) break;
    }
    __syncwarp();
    if (fix_k_tail) {
      const int j = nkb - 1, s = j % C::kStagesK;
      if (mbar_wait_warp(&bars->a_full[s], (j / C::kStagesK) & 1, ctx)) {
        zero_tile_rows_from<D>(sK + s * C::kTileBytes, sk - j * kBlock, lane);
        if (lane == 0) mbar_arrive(&bars->tail_fixed[0]);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_nn = make_idesc_f16(128, kBlock, false, false);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      // S(j+1) is issued as soon as S(j) sits in registers and dP(j+1) as soon as dP(j) does, so both run
      // under the elementwise work of block j.  The hooks wait for the TMA load the next product reads.
      auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, ctx); };
      auto k_tile = [&](int j) { return smem_u32(sK + (j % C::kStagesK) * C::kTileBytes); };
      auto v_tile = [&](int j) { return smem_u32(sV + (j % C::kStagesV) * C::kTileBytes); };
      auto k_full = [&](int j) { return wait(&bars->a_full[j % C::kStagesK], (j / C::kStagesK) & 1); };
      auto v_full = [&](int j) { return wait(&bars->b_full[j % C::kStagesV], (j / C::kStagesV) & 1); };
      bool ok = wait(&bars->fixed_full, 0) && k_full(0);
      for (int j = 0; ok && j < nb; ++j) {
        if (j > 0 && !(ok = wait(&bars->s_loaded, (j - 1) & 1))) break;
        // S(j) complete tells the elementwise warps that packed-dS buffer j&1 is free again
        if (j >= 2 && !(ok = wait(&bars->ds_free[j & 1], ((j >> 1) - 1) & 1))) break;
        tc_fence_after_sync();
        ok = gemm_ss<D>(tmem_base + kColS, q_addr, k_tile(j), idesc_nn, [&] { return v_full(j); });
        if (!ok) break;
        tc_commit(&bars->s_full);
        tc_commit(&bars->a_empty[j % C::kStagesK]);  // second reader: the dQ MMAs of this block
        if (j > 0 && !(ok = wait(&bars->dp_loaded, (j - 1) & 1))) break;
        tc_fence_after_sync();
        ok = gemm_ss<D>(tmem_base + kColDP, do_addr, v_tile(j), idesc_nn,
                        [&] { return j + 1 >= nb || k_full(j + 1); });
        if (!ok) break;
        tc_commit(&bars->dp_full);
        tc_commit(&bars->b_empty[j % C::kStagesV]);
      }
    }
  } else if (warp == kAccMmaWarp) {
    if (lane == 0 && nb > 0) {
      // dQ += dS(j) K(j) as soon as the packed dS(j) is written.  dS has two buffers; ds_free[u] tells the
      // elementwise warps that buffer u has been consumed.
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, false, true);
      bool ok = true;
      for (int j = 0; ok && j < nb; ++j) {
        const int s = j % C::kStagesK;
        if (!(ok = mbar_wait(&bars->a_full[s], (j / C::kStagesK) & 1, ctx))) break;
        if (!(ok = mbar_wait(&bars->ds_full, j & 1, ctx))) break;
        if (fix_k_tail && j == nkb - 1 && !(ok = mbar_wait(&bars->tail_fixed[0], 0, ctx))) break;
        tc_fence_after_sync();
        gemm_ts<D>(tmem_base + kColAcc, tmem_base + kColPacked + (j & 1) * 64, smem_u32(sK + s * C::kTileBytes),
                   idesc_acc, j == 0);
        tc_commit(&bars->a_empty[s]);
        tc_commit(&bars->ds_free[j & 1]);
      }
      if (ok) tc_commit(&bars->acc_full);
    }
  } else {
    // ---- elementwise warps: thread = (row, 32-column quarter) ----
    const int cq = warp >> 2, quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int row = row0 + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + cq * 32;
    const uint32_t tDP = tmem_base + lane_base + kColDP + cq * 32;
    const int64_t stat_idx = (static_cast<int64_t>(batch) * p.h + head) * p.sq_pad + row;
    const float neg_lse2 = p.lse2[stat_idx];
    const float neg_delta = p.delta[stat_idx];
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c), nl2 = make_float2(neg_lse2, neg_lse2), nd2 = make_float2(neg_delta, neg_delta);
    bool ok = true;
    bool s_ready = false;  // probe of s_full for the coming block
    for (int j = 0; j < nb; ++j) {
      if (!(ok = warp_wait_unless(s_ready, &bars->s_full, j & 1, ctx))) break;
      tc_fence_after_sync();
      uint32_t sr[32];
      tmem_ld32(tS, sr);
      const bool dp_ready = warp_probe(&bars->dp_full, j & 1);  // dP(j) follows S(j) through the pipe
      tmem_wait_ld();
      warp_arrive_loaded(&bars->s_loaded, lane);
      const int col0 = j * kBlock + cq * 32;
      int limit = sk - 1 - col0;
      if (p.is_causal) limit = min(limit, row + sk - sq - col0);
      float2 pr[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 x = ffma2(make_float2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), c2, nl2);
        pr[i] = exp2_pair(x);
      }
      if (limit < 31) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (2 * i > limit) pr[i].x = 0.f;
          if (2 * i + 1 > limit) pr[i].y = 0.f;
        }
      }
      if (!(ok = warp_wait_unless(dp_ready, &bars->dp_full, j & 1, ctx))) break;
      tc_fence_after_sync();
      tmem_ld32(tDP, sr);
      s_ready = j + 1 < nb && warp_probe(&bars->s_full, (j + 1) & 1);  // S(j+1) ran under the exponentials
      tmem_wait_ld();
      warp_arrive_loaded(&bars->dp_loaded, lane);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 d = fmul2(pr[i], fadd2(make_float2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), nd2));
        pk[i] = pack_half2(d.x, d.y);
      }
      if (limit < 31) {  // by selection: dP of a masked column may be NaN/Inf (rows of the next sequence in V)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (2 * i > limit) pk[i] &= 0xffff0000u;
          if (2 * i + 1 > limit) pk[i] &= 0x0000ffffu;
        }
      }
      // packed dS: 64 consecutive columns per block (16 per column quarter), two alternating buffers; the
      // buffer is free because S(j) was issued only after the dQ MMAs of block j-2 had consumed it
      tmem_st16(tmem_base + lane_base + kColPacked + (j & 1) * 64 + cq * 16, pk);
      warp_arrive(&bars->ds_full, lane);
    }
    // ---- epilogue: dQ = scale * acc; D/32 of the 16 warps-per-lane-quarter groups store 32 columns each ----
    const bool stores = cq < D / 32;
    const int64_t dq_idx = (varlen ? static_cast<int64_t>(q_off + row) * p.dq_row_stride
                                   : batch * p.dq_batch_stride + static_cast<int64_t>(row) * p.dq_row_stride) +
                           head * p.dq_head_stride + cq * 32;
    if (ok && nb > 0) ok = mbar_wait_warp(&bars->acc_full, 0, ctx);
    if (ok && stores) {
      if (nb > 0) {
        tc_fence_after_sync();
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + kColAcc + cq * 32, r);
        tmem_wait_ld();
        if (row < sq) store_row_fp16(p.dq + dq_idx, r, p.scale);
      } else if (row < sq) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(p.dq + dq_idx + i * 8) = z;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// =============================================================================================
// 3. dK/dV kernel
// =============================================================================================
// kVarlen: the sequences are packed (cu_seqlens); only then can a Q tile hold rows of a neighbouring
// sequence, and only that instantiation carries the code that guards against them.
template <int D, bool kVarlen>
__global__ void __launch_bounds__(kNumThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ BwdKernelParams p) {
  using C = BCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int batch = blockIdx.z, head_k = blockIdx.y, nblk = blockIdx.x;
  constexpr bool varlen = kVarlen;
  const int q_off = varlen ? p.cu_seqlens_q[batch] : 0;
  const int sq = varlen ? p.cu_seqlens_q[batch + 1] - q_off : p.seqlen_q;
  const int k_off = varlen ? p.cu_seqlens_k[batch] : 0;
  const int sk = varlen ? p.cu_seqlens_k[batch + 1] - k_off : p.seqlen_k;
  const int key0 = nblk * kBlock;
  if (key0 >= sk) return;
  if (p.status && (*reinterpret_cast<volatile int*>(p.status) & kStatusWaitTimeout) != 0) return;
  const int bq = varlen ? 0 : batch;
  const int group = p.h / p.h_k;
  const int nq = (sq + kBlock - 1) / kBlock;
  int i_min = 0;
  if (p.is_causal) {
    const int first_row = key0 - (sk - sq);  // first query row that can see key0
    i_min = first_row <= 0 ? 0 : first_row / kBlock;
  }
  const int per_head = max(0, nq - i_min);
  const int n_it = per_head * group;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::kTileBytes;
  uint8_t* sQ = sV + C::kTileBytes;
  uint8_t* sdO = sQ + C::kStagesQ * C::kTileBytes;
  float* sStats = reinterpret_cast<float*>(sdO + C::kStagesDO * C::kTileBytes);  // [2][lse2 128 | delta 128]
  BBarriers* bars = reinterpret_cast<BBarriers*>(reinterpret_cast<uint8_t*>(sStats) + 2048);
  static_assert(sizeof(BBarriers) <= 512, "barrier block");
  if (smem - smem_raw > C::kAlignPadDkdv) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusSmemLayout);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The TMA producer thread initialises the barriers itself and issues the loads of K, V and of the first
  // Q / statistics / dO tiles BEFORE the CTA-wide synchronisation, so that their latency overlaps the TMEM
  // allocation.
  WaitCtx ctx{&bars->abort_flag, p.status};
  auto load_q_do = [&](int it) -> bool {
    const int sq_ = it % C::kStagesQ, sd = it % C::kStagesDO, ss = it & 1;
    const uint32_t phq = (it / C::kStagesQ) & 1, phd = (it / C::kStagesDO) & 1, phs = (it >> 1) & 1;
    const int head = head_k * group + it / per_head;
    const int i = i_min + it % per_head;
    const int qrow = q_off + i * kBlock;
    const int64_t stat = (static_cast<int64_t>(batch) * p.h + head) * p.sq_pad + i * kBlock;
    if (!mbar_wait(&bars->a_empty[sq_], phq ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->a_full[sq_], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sQ + sq_ * C::kTileBytes + c * C::kChunkBytes, &p.tm_q, &bars->a_full[sq_], c * 64, head, qrow, bq);
    if (!mbar_wait(&bars->st_empty[ss], phs ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->st_full[ss], 1024);
    bulk_load_1d(sStats + ss * 256, p.lse2 + stat, 512, &bars->st_full[ss]);
    bulk_load_1d(sStats + ss * 256 + 128, p.delta + stat, 512, &bars->st_full[ss]);
    if (!mbar_wait(&bars->b_empty[sd], phd ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->b_full[sd], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sdO + sd * C::kTileBytes + c * C::kChunkBytes, &p.tm_do, &bars->b_full[sd], c * 64, head, qrow, bq);
    return true;
  };
  const int n_early = min(n_it, 2);  // stages that are free from the start: no wait blocks
  if (warp == kProducerWarp && lane == 0) {
    init_barriers(bars, C::kStagesQ, 2, 2);
    if (n_it > 0) {
      mbar_arrive_expect_tx(&bars->fixed_full, 2 * C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(sK + c * C::kChunkBytes, &p.tm_k, &bars->fixed_full, c * 64, head_k, k_off + key0, bq);
        tma_load_4d(sV + c * C::kChunkBytes, &p.tm_v, &bars->fixed_full, c * 64, head_k, k_off + key0, bq);
      }
      for (int it = 0; it < n_early; ++it) load_q_do(it);
    }
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  // the last Q / dO tile of a packed sequence holds rows of the next sequence (see zero_tile_rows_from)
  const bool fix_q_tail = kVarlen && (sq % kBlock) != 0 && n_it > 0;
  const int q_tail_rows = sq - (nq - 1) * kBlock;  // valid rows of the last Q tile
  if (warp == kProducerWarp) {
    if (!fix_q_tail) {
      if (lane == 0) {
        for (int it = n_early; it < n_it; ++it)
          if (!load_q_do(it)) break;
      }
    } else {
      // the whole warp walks the tiles: lane 0 issues the loads, all lanes zero the tails
      for (int it = 0; it < n_it; ++it) {
        bool loaded = true;
        if (lane == 0 && it >= n_early) loaded = load_q_do(it);
        if (!__shfl_sync(0xffffffffu, loaded, 0)) break;
        if (it % per_head == per_head - 1) {  // the last Q tile of this head
          const int sq_ = it % C::kStagesQ, sd = it % C::kStagesDO;
          if (!mbar_wait_warp(&bars->a_full[sq_], (it / C::kStagesQ) & 1, ctx)) break;
          if (!mbar_wait_warp(&bars->b_full[sd], (it / C::kStagesDO) & 1, ctx)) break;
          zero_tile_rows_from<D>(sQ + sq_ * C::kTileBytes, q_tail_rows, lane);
          zero_tile_rows_from<D>(sdO + sd * C::kTileBytes, q_tail_rows, lane);
          if (lane == 0) mbar_arrive(&bars->tail_fixed[sd]);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_nn = make_idesc_f16(128, kBlock, false, false);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      // One accumulator region A holds S^T(it) and then dP^T(it): dP^T(it) is issued as soon as S^T(it)
      // sits in registers, S^T(it+1) as soon as dP^T(it) does.  The hooks wait for the TMA load the next
      // product reads.
      auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, ctx); };
      auto q_tile = [&](int it) { return smem_u32(sQ + (it % C::kStagesQ) * C::kTileBytes); };
      auto do_tile = [&](int it) { return smem_u32(sdO + (it % C::kStagesDO) * C::kTileBytes); };
      auto q_full = [&](int it) { return wait(&bars->a_full[it % C::kStagesQ], (it / C::kStagesQ) & 1); };
      auto do_full = [&](int it) { return wait(&bars->b_full[it % C::kStagesDO], (it / C::kStagesDO) & 1); };
      const uint32_t tA = tmem_base + kColS, tA2 = tmem_base + kColDPT<D>;
      constexpr bool kSharedRegion = kColDPT<D> == kColS;
      bool ok = wait(&bars->fixed_full, 0) && q_full(0);
      for (int it = 0; ok && it < n_it; ++it) {
        // region A is free once its last content was read: dP^T(it-1) when the region is shared, S^T(it-1) otherwise
        if (it > 0 && !(ok = wait(kSharedRegion ? &bars->dp_loaded : &bars->s_loaded, (it - 1) & 1))) break;
        tc_fence_after_sync();
        ok = gemm_ss<D>(tA, k_addr, q_tile(it), idesc_nn, [&] { return do_full(it); });  // S^T(it) = K Q^T
        if (!ok) break;
        tc_commit(&bars->s_full);
        tc_commit(&bars->a_empty[it % C::kStagesQ]);  // second reader: the dK MMAs of this tile
        // the region of dP^T is free once S^T(it) (shared) or dP^T(it-1) (own region) was read
        if (kSharedRegion) {
          if (!(ok = wait(&bars->s_loaded, it & 1))) break;
        } else if (it > 0) {
          if (!(ok = wait(&bars->dp_loaded, (it - 1) & 1))) break;
        }
        tc_fence_after_sync();
        ok = gemm_ss<D>(tA2, v_addr, do_tile(it), idesc_nn,  // dP^T(it) = V dO^T
                        [&] { return it + 1 >= n_it || q_full(it + 1); });
        if (!ok) break;
        tc_commit(&bars->dp_full);
        tc_commit(&bars->b_empty[it % C::kStagesDO]);  // second reader: the dV MMAs of this tile
      }
    }
  } else if (warp == kAccMmaWarp) {
    if (lane == 0 && n_it > 0) {
      // dV += P^T(it) dO(it) as soon as the packed P^T is written, dK += dS^T(it) Q(it) likewise.
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, false, true);
      const uint32_t tP = tmem_base + kColDP, tDS = tmem_base + kColDP + 64;
      const uint32_t tDV = tmem_base + kColAcc, tDK = tmem_base + kColAcc + D;
      bool ok = true;
      uint32_t tail_phase = 0;  // bit sd: parity of the next tail_fixed[sd] phase to wait for
      for (int it = 0; ok && it < n_it; ++it) {
        const int sq_ = it % C::kStagesQ, sd = it % C::kStagesDO;
        if (!(ok = mbar_wait(&bars->b_full[sd], (it / C::kStagesDO) & 1, ctx))) break;
        if (!(ok = mbar_wait(&bars->p_full, it & 1, ctx))) break;
        if (fix_q_tail && it % per_head == per_head - 1) {
          if (!(ok = mbar_wait(&bars->tail_fixed[sd], (tail_phase >> sd) & 1, ctx))) break;
          tail_phase ^= 1u << sd;
        }
        tc_fence_after_sync();
        gemm_ts<D>(tDV, tP, smem_u32(sdO + sd * C::kTileBytes), idesc_acc, it == 0);
        tc_commit(&bars->b_empty[sd]);
        tc_commit(&bars->p_free);
        if (!(ok = mbar_wait(&bars->a_full[sq_], (it / C::kStagesQ) & 1, ctx))) break;
        if (!(ok = mbar_wait(&bars->ds_full, it & 1, ctx))) break;
        tc_fence_after_sync();
        gemm_ts<D>(tDK, tDS, smem_u32(sQ + sq_ * C::kTileBytes), idesc_acc, it == 0);
        tc_commit(&bars->a_empty[sq_]);
        tc_commit(&bars->ds_free[0]);
      }
      if (ok) tc_commit(&bars->acc_full);
    }
  } else {
    // ---- elementwise warps: thread = (key row, 32-query-column quarter) ----
    const int cq = warp >> 2, quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int key = key0 + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tA = tmem_base + lane_base + kColS + cq * 32;         // S^T, then dP^T
    const uint32_t tP = tmem_base + lane_base + kColDP + cq * 16;        // packed P^T
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    // causal: query column q of tile i is masked for this key when key > q + sk - sq, i.e. the columns of
    // this thread's quarter below  key - (sk - sq) - (i * 128 + cq * 32)  are masked
    const int cmin0 = p.is_causal ? key - (sk - sq) - (i_min * kBlock + cq * 32) : 0;
    const float* stats = sStats + cq * 32;
    const int cmax_last = fix_q_tail ? max(0, min(32, q_tail_rows - cq * 32)) : 32;  // valid columns in the last Q tile
    int i_rel = 0;  // Q tile within the current head
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int ss = it & 1;
      if (!(ok = mbar_wait_warp(&bars->st_full[ss], (it >> 1) & 1, ctx))) break;
      // D = 128: the LSE of this thread's 32 query columns is fetched while the warp waits for S^T anyway.
      // Read after the wait, these shared-memory loads compete with the operand fetches of the dP^T MMAs, which
      // take the whole shared-memory bandwidth (measured: 4.5-7 % of the kernel; at D = 64 the MMAs are half as
      // long and the early loads cost 2 % instead).
      const float4* st_lse = reinterpret_cast<const float4*>(stats + ss * 256);
      const float4* st_delta = reinterpret_cast<const float4*>(stats + ss * 256 + 128);
      constexpr bool kEarlyLse = (D == 128);
      float4 lse_q[8];
      if constexpr (kEarlyLse) {
#pragma unroll
        for (int e = 0; e < 8; ++e) lse_q[e] = st_lse[e];
      }
      if (!(ok = mbar_wait_warp(&bars->s_full, it & 1, ctx))) break;
      tc_fence_after_sync();
      uint32_t sr[32];
      tmem_ld32(tA, sr);
      tmem_wait_ld();
      warp_arrive_loaded(&bars->s_loaded, lane);  // region A may now receive dP^T
      // columns below cmin are masked by causality; columns from cmax on are query rows past the end of the
      // sequence (last Q tile of a packed sequence).  Both clamped to [0, 32] and packed into one register.
      const int cmask = max(0, min(32, cmin0 - i_rel * kBlock)) |
                        (((kVarlen && i_rel == per_head - 1) ? cmax_last : 32) << 8);
      const bool col_masked = cmask != (32 << 8);
      if (++i_rel == per_head) i_rel = 0;
      float2 pr[16];
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float4 l = kEarlyLse ? lse_q[e] : st_lse[e];
        pr[2 * e] = exp2_pair(ffma2(make_float2(__uint_as_float(sr[4 * e]), __uint_as_float(sr[4 * e + 1])), c2,
                                    make_float2(l.x, l.y)));
        pr[2 * e + 1] = exp2_pair(ffma2(make_float2(__uint_as_float(sr[4 * e + 2]), __uint_as_float(sr[4 * e + 3])),
                                        c2, make_float2(l.z, l.w)));
      }
      if (col_masked) {
        const int cmin = cmask & 0xff, cmax = cmask >> 8;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (2 * e < cmin || 2 * e >= cmax) pr[e].x = 0.f;
          if (2 * e + 1 < cmin || 2 * e + 1 >= cmax) pr[e].y = 0.f;
        }
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) pk[e] = pack_half2(pr[e].x, pr[e].y);
      // the dV MMAs of the previous tile must have consumed the old P^T before it is overwritten
      if (it > 0 && !(ok = mbar_wait_warp(&bars->p_free, (it - 1) & 1, ctx))) break;
      tmem_st16(tP, pk);
      warp_arrive(&bars->p_full, lane);

      if (!(ok = mbar_wait_warp(&bars->dp_full, it & 1, ctx))) break;
      tc_fence_after_sync();
      tmem_ld32(tA + (kColDPT<D> - kColS), sr);
      tmem_wait_ld();
      warp_arrive_loaded(&bars->dp_loaded, lane);  // region A may now receive the next S^T
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float4 dl = st_delta[e];
        const float2 d0 = fmul2(pr[2 * e], fadd2(make_float2(__uint_as_float(sr[4 * e]), __uint_as_float(sr[4 * e + 1])),
                                                 make_float2(dl.x, dl.y)));
        const float2 d1 = fmul2(pr[2 * e + 1], fadd2(make_float2(__uint_as_float(sr[4 * e + 2]), __uint_as_float(sr[4 * e + 3])),
                                                     make_float2(dl.z, dl.w)));
        pk[2 * e] = pack_half2(d0.x, d0.y);
        pk[2 * e + 1] = pack_half2(d1.x, d1.y);
      }
      if (col_masked) {  // by selection: dP^T of a masked column may be NaN/Inf (dO rows of the next sequence)
        const int cmin = cmask & 0xff, cmax = cmask >> 8;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (2 * e < cmin || 2 * e >= cmax) pk[e] &= 0xffff0000u;
          if (2 * e + 1 < cmin || 2 * e + 1 >= cmax) pk[e] &= 0x0000ffffu;
        }
      }
      // the statistics of this tile are in use no longer
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->st_empty[ss]);
      if (it > 0 && !(ok = mbar_wait_warp(&bars->ds_free[0], (it - 1) & 1, ctx))) break;
      tmem_st16(tP + 64, pk);  // packed dS^T
      warp_arrive(&bars->ds_full, lane);
    }
    // ---- epilogue: column quarters 0,1 store the halves of dV, quarters 2,3 the halves of dK * scale ----
    const int which = cq >> 1;        // 0 = dV, 1 = dK
    const int col_half = cq & 1;      // which D/2 columns
    __half* dst_base = (which == 0) ? p.dv : p.dk;
    const int64_t bs = (which == 0) ? p.dv_batch_stride : p.dk_batch_stride;
    const int64_t rs = (which == 0) ? p.dv_row_stride : p.dk_row_stride;
    const int64_t hs = (which == 0) ? p.dv_head_stride : p.dk_head_stride;
    __half* dst = dst_base + (varlen ? static_cast<int64_t>(k_off + key) * rs : batch * bs + static_cast<int64_t>(key) * rs) +
                  head_k * hs + col_half * (D / 2);
    const float mul = (which == 0) ? 1.f : p.scale;
    if (ok && n_it > 0) ok = mbar_wait_warp(&bars->acc_full, 0, ctx);
    if (ok) {
      if (n_it > 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < D / 64; ++q) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_base + kColAcc + which * D + col_half * (D / 2) + q * 32, r);
          tmem_wait_ld();
          if (key < sk) store_row_fp16(dst + q * 32, r, mul);
        }
      } else if (key < sk) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i3 = 0; i3 < D / 16; ++i3) *reinterpret_cast<uint4*>(dst + i3 * 8) = z;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

int round_up(int x, int m) { return (x + m - 1) / m * m; }

size_t stats_floats(const FaBwdParams* p) {
  return static_cast<size_t>(p->b) * p->h * round_up(p->seqlen_q, kBlock);
}

template <int D>
int launch_bwd(const BwdKernelParams& kp, const FaBwdParams* p, int stage_mask, cudaStream_t stream) {
  using C = BCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesDq));
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dkdv_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesDkdv));
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dkdv_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesDkdv));
    configured[dev & 63] = true;
  }
  if (stage_mask & 2) {
    dim3 grid_q((p->seqlen_q + kBlock - 1) / kBlock, p->h, p->b);
    bwd_dq_kernel<D><<<grid_q, kNumThreads, C::kSmemBytesDq, stream>>>(kp);
    FA_CHECK_CUDA(cudaGetLastError());
  }
  if (stage_mask & 4) {
    dim3 grid_k((p->seqlen_k + kBlock - 1) / kBlock, p->h_k, p->b);
    if (kp.cu_seqlens_q != nullptr)
      bwd_dkdv_kernel<D, true><<<grid_k, kNumThreads, C::kSmemBytesDkdv, stream>>>(kp);
    else
      bwd_dkdv_kernel<D, false><<<grid_k, kNumThreads, C::kSmemBytesDkdv, stream>>>(kp);
    FA_CHECK_CUDA(cudaGetLastError());
  }
  return FA_OK;
}

}  // namespace
}  // namespace fa

extern "C" size_t fa_bwd_workspace_bytes(const FaBwdParams* p) {
  if (p == nullptr || p->b < 1 || p->h < 1 || p->seqlen_q < 1) return 0;
  return 2 * fa::stats_floats(p) * sizeof(float);
}

extern "C" int fa_bwd(const FaBwdParams* p, fa_stream_t stream) { return fa_bwd_stages(p, 7, stream); }

extern "C" int fa_bwd_stages(const FaBwdParams* p, int stage_mask, fa_stream_t stream_) {
  using namespace fa;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  FA_CHECK_ARG(p != nullptr, "fa_bwd: params is NULL");
  FA_CHECK_ARG(p->q && p->k && p->v && p->o && p->dout && p->lse && p->dq && p->dk && p->dv,
               "fa_bwd: q, k, v, o, dout, lse, dq, dk, dv must be non-NULL");
  if (p->d != 64 && p->d != 128) return set_error(FA_ERR_UNSUPPORTED, "fa_bwd: head_dim must be 64 or 128");
  FA_CHECK_ARG(p->b >= 1 && p->h >= 1 && p->h_k >= 1 && p->h % p->h_k == 0, "fa_bwd: bad b / h / h_k");
  FA_CHECK_ARG(p->seqlen_q >= 1 && p->seqlen_k >= 1, "fa_bwd: bad sequence lengths");
  FA_CHECK_ARG((p->cu_seqlens_q == nullptr) == (p->cu_seqlens_k == nullptr),
               "fa_bwd: cu_seqlens_q and cu_seqlens_k go together");
  FA_CHECK_ARG(p->lse_row_stride >= p->seqlen_q, "fa_bwd: lse_row_stride is smaller than seqlen_q");
  const bool varlen = p->cu_seqlens_q != nullptr;
  {
    const void* ptrs[] = {p->o, p->dout, p->dq, p->dk, p->dv};
    for (const void* x : ptrs) FA_CHECK_ARG(aligned16(x), "fa_bwd: o, dout, dq, dk, dv must be 16-byte aligned");
    const int64_t strides[] = {p->o_row_stride,  p->o_head_stride,  p->do_row_stride, p->do_head_stride,
                               p->dq_row_stride, p->dq_head_stride, p->dk_row_stride, p->dk_head_stride,
                               p->dv_row_stride, p->dv_head_stride};
    for (int64_t s : strides) FA_CHECK_ARG(s % 8 == 0, "fa_bwd: strides must be multiples of 8 elements");
    if (!varlen) {
      const int64_t bs[] = {p->o_batch_stride, p->do_batch_stride, p->dq_batch_stride, p->dk_batch_stride,
                            p->dv_batch_stride};
      for (int64_t s : bs) FA_CHECK_ARG(s % 8 == 0, "fa_bwd: batch strides must be multiples of 8 elements");
    }
  }
  const size_t need = fa_bwd_workspace_bytes(p);
  if (p->workspace == nullptr || p->workspace_bytes < need)
    return set_error(FA_ERR_WORKSPACE, "fa_bwd: workspace smaller than fa_bwd_workspace_bytes()");
  FA_CHECK_ARG(aligned16(p->workspace), "fa_bwd: workspace must be 16-byte aligned");
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;

  const int sq_pad = round_up(p->seqlen_q, kBlock);
  float* delta = static_cast<float*>(p->workspace);
  float* lse2 = delta + stats_floats(p);

  PreParams pp;
  pp.o = static_cast<const __half*>(p->o);
  pp.dout = static_cast<const __half*>(p->dout);
  pp.lse = p->lse;
  pp.delta = delta;
  pp.lse2 = lse2;
  pp.o_batch_stride = p->o_batch_stride; pp.o_row_stride = p->o_row_stride; pp.o_head_stride = p->o_head_stride;
  pp.do_batch_stride = p->do_batch_stride; pp.do_row_stride = p->do_row_stride; pp.do_head_stride = p->do_head_stride;
  pp.lse_row_stride = p->lse_row_stride;
  pp.h = p->h; pp.seqlen_q = p->seqlen_q; pp.sq_pad = sq_pad; pp.d = p->d;
  pp.cu_seqlens_q = p->cu_seqlens_q;
  const int64_t pre_items = static_cast<int64_t>((sq_pad + kPreRows - 1) / kPreRows) * p->h;
  const int items_per_block = 256 / (p->d / 8);
  dim3 grid_pre(static_cast<unsigned>((pre_items + items_per_block - 1) / items_per_block), 1, p->b);
  if (stage_mask & 1) {
    bwd_preprocess_kernel<<<grid_pre, 256, 0, stream>>>(pp);
    FA_CHECK_CUDA(cudaGetLastError());
  }

  BwdKernelParams kp;
  const int64_t q_rows = varlen ? p->total_q : p->seqlen_q;
  const int64_t k_rows = varlen ? p->total_k : p->seqlen_k;
  const int64_t nb = varlen ? 1 : p->b;
  FA_CHECK_ARG(q_rows >= 1 && k_rows >= 1, "fa_bwd: empty q or k");
  rc = make_tensor_map_4d(&kp.tm_q, p->q, p->d, p->h, q_rows, nb, p->q_head_stride, p->q_row_stride,
                          p->q_batch_stride, kBlock, "fa_bwd: q");
  if (rc != FA_OK) return rc;
  rc = make_tensor_map_4d(&kp.tm_do, p->dout, p->d, p->h, q_rows, nb, p->do_head_stride, p->do_row_stride,
                          p->do_batch_stride, kBlock, "fa_bwd: dout");
  if (rc != FA_OK) return rc;
  rc = make_tensor_map_4d(&kp.tm_k, p->k, p->d, p->h_k, k_rows, nb, p->k_head_stride, p->k_row_stride,
                          p->k_batch_stride, kBlock, "fa_bwd: k");
  if (rc != FA_OK) return rc;
  rc = make_tensor_map_4d(&kp.tm_v, p->v, p->d, p->h_k, k_rows, nb, p->v_head_stride, p->v_row_stride,
                          p->v_batch_stride, kBlock, "fa_bwd: v");
  if (rc != FA_OK) return rc;
  kp.dq = static_cast<__half*>(p->dq);
  kp.dk = static_cast<__half*>(p->dk);
  kp.dv = static_cast<__half*>(p->dv);
  kp.dq_batch_stride = p->dq_batch_stride; kp.dq_row_stride = p->dq_row_stride; kp.dq_head_stride = p->dq_head_stride;
  kp.dk_batch_stride = p->dk_batch_stride; kp.dk_row_stride = p->dk_row_stride; kp.dk_head_stride = p->dk_head_stride;
  kp.dv_batch_stride = p->dv_batch_stride; kp.dv_row_stride = p->dv_row_stride; kp.dv_head_stride = p->dv_head_stride;
  kp.delta = delta;
  kp.lse2 = lse2;
  kp.sq_pad = sq_pad;
  kp.seqlen_q = p->seqlen_q; kp.seqlen_k = p->seqlen_k; kp.h = p->h; kp.h_k = p->h_k;
  kp.scale = p->softmax_scale;
  kp.scale_log2 = p->softmax_scale * kLog2e;
  kp.is_causal = p->is_causal;
  kp.cu_seqlens_q = p->cu_seqlens_q;
  kp.cu_seqlens_k = p->cu_seqlens_k;
  kp.status = device_status_ptr();
  if (p->d == 128) return launch_bwd<128>(kp, p, stage_mask, stream);
  return launch_bwd<64>(kp, p, stage_mask, stream);
}
