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
#include "bwd_common.cuh"

namespace fa {
namespace {

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
// A work item is one 128-row Q tile of one (sequence, query head): S = Q K^T and dP = dO V^T per key block (SS),
// P and dS in the elementwise warps, dQ += dS K (TS, A = packed dS in TMEM, two alternating buffers).  The kernel
// is persistent: one CTA per SM takes items from a global counter (heaviest causal tile of a head first) and
// keeps its barriers, its TMEM allocation and the K / V rings across items: every barrier phase is derived from
// the cumulative block count G (or the item count), the Q / dO tiles and the row statistics of the next item are
// loaded as soon as the last dP product of the current item has read them, and the first S product of the next
// item is issued under the last elementwise block and the epilogue of the current one.  The row statistics come
// through shared memory with the Q / dO tiles (no global load at the start of an item).  Scheduling as in the
// forward kernel: an item is claimed two blocks before the current one ends.  Measured against one CTA per item
// (bit-identical results): S = 8192 1.4 % faster, S = 4096 5 %, S = 1024 19 %, D = 64 S = 4096 11 %.
constexpr int kDqpThreads = 640;  // + one scheduler warp: 20 warps, five on one sub-partition -> 96 registers
constexpr int kDqpSchedWarp = 19;
constexpr int kDqpReaders = kComputeWarps + 3;  // elementwise warps, producer warp, two MMA threads
static_assert((kDqpThreads / 32 + 3) / 4 * 32 * 96 <= 16384, "register file of one SM sub-partition");

struct DqpItem {
  int batch, head, mblk, pad;  // mblk < 0: no more work
};
struct DqpBarriers {
  BBarriers b;
  uint64_t q_free;          // the Q / dO tiles and the statistics of the item have been read for the last time
  uint64_t sched_full[2], sched_empty[2], sched_go;
  DqpItem items[2];
};
static_assert(sizeof(DqpBarriers) <= 512, "barrier block");

struct DqpWork {
  int batch, head, head_k, bq, q_off, k_off, sq, sk, row0, nkb, nb, shift;
  bool fix_k_tail;
};
__device__ __forceinline__ DqpWork dqp_decode(const BwdKernelParams& p, const DqpItem& it) {
  DqpWork w;
  const bool varlen = p.cu_seqlens_q != nullptr;
  w.batch = it.batch, w.head = it.head;
  w.q_off = varlen ? p.cu_seqlens_q[it.batch] : 0;
  w.sq = varlen ? p.cu_seqlens_q[it.batch + 1] - w.q_off : p.seqlen_q;
  w.k_off = varlen ? p.cu_seqlens_k[it.batch] : 0;
  w.sk = varlen ? p.cu_seqlens_k[it.batch + 1] - w.k_off : p.seqlen_k;
  w.row0 = it.mblk * kBlock;
  w.bq = varlen ? 0 : it.batch;
  w.head_k = it.head / (p.h / p.h_k);
  w.nkb = (w.sk + kBlock - 1) / kBlock;
  w.shift = (p.is_causal == 2) ? p.causal_shift : w.sk - w.sq;
  w.nb = w.nkb;
  if (p.is_causal) {
    const int x = w.row0 + kBlock + w.shift;
    w.nb = x <= 0 ? 0 : min(w.nkb, (x + kBlock - 1) / kBlock);
  }
  w.fix_k_tail = varlen && (w.sk % kBlock) != 0 && w.nb == w.nkb && w.nb > 0;
  return w;
}

template <int D>
__global__ void __launch_bounds__(kDqpThreads, 1)
bwd_dq_kernel(const __grid_constant__ BwdKernelParams p) {
  using C = BCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const int stop_probe = stop_probe_begin(p.status);

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::kTileBytes;
  uint8_t* sK = sdO + C::kTileBytes;
  uint8_t* sV = sK + C::kStagesK * C::kTileBytes;
  float* sStats = reinterpret_cast<float*>(sV + C::kStagesV * C::kTileBytes);  // lse2[128] | delta[128]
  DqpBarriers* xb = reinterpret_cast<DqpBarriers*>(reinterpret_cast<uint8_t*>(sStats) + 1024);
  BBarriers* bars = &xb->b;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == kProducerWarp && lane == 0) {
    init_barriers(bars, C::kStagesK, 2, 1);
    mbar_init(&xb->q_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&xb->sched_full[i], 1);
      mbar_init(&xb->sched_empty[i], kDqpReaders);
    }
    mbar_init(&xb->sched_go, 1);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  const bool stop = __syncthreads_or(stop_probe) != 0;
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  WaitCtx ctx{&bars->abort_flag, p.status};

  auto read_item = [&](int n, DqpItem& it) -> bool {
    if (!mbar_wait(&xb->sched_full[n & 1], (n >> 1) & 1, ctx)) return false;
    it = xb->items[n & 1];
    return true;
  };
  auto release_item = [&](int n) { mbar_arrive(&xb->sched_empty[n & 1]); };

  if (stop) {
  } else if (warp == kDqpSchedWarp) {
    if (lane == 0) {
      bool finished = false;
      int seq = 0;
      for (int n = 0;; ++n) {
        int next = blockIdx.x;
        if (n > 0) {
          if (!mbar_wait(&xb->sched_go, (n - 1) & 1, ctx)) break;
          next = gridDim.x + atomicAdd(p.sched, 1);
        }
        DqpItem it;
        it.batch = 0, it.head = 0, it.mblk = -1, it.pad = 0;
        while (next < p.total_items) {
          int batch, head, mblk, sq;
          if (p.cu_seqlens_q == nullptr) {
            const int x = next % p.items_x, rest = next / p.items_x;
            head = rest % p.h, batch = rest / p.h, mblk = p.items_x - 1 - x, sq = p.seqlen_q;
          } else {  // slots per sequence from cu_seqlens_q / 128 (at most one spare slot per sequence and head)
            while (seq + 1 < p.b && p.h * ((p.cu_seqlens_q[seq + 1] >> 7) + seq + 1) <= next) ++seq;
            const int v0 = (p.cu_seqlens_q[seq] >> 7) + seq, v1 = (p.cu_seqlens_q[seq + 1] >> 7) + seq + 1;
            const int rel = next - p.h * v0, cnt = v1 - v0;
            sq = p.cu_seqlens_q[seq + 1] - p.cu_seqlens_q[seq];
            batch = seq, head = rel / cnt, mblk = (sq + kBlock - 1) / kBlock - 1 - rel % cnt;
            if (head >= p.h) mblk = -1;
          }
          if (mblk >= 0 && mblk * kBlock < sq) {
            it.batch = batch, it.head = head, it.mblk = mblk;
            break;
          }
          next = gridDim.x + atomicAdd(p.sched, 1);
        }
        if (!mbar_wait(&xb->sched_empty[n & 1], ((n >> 1) & 1) ^ 1, ctx)) break;
        xb->items[n & 1] = it;
        mbar_arrive(&xb->sched_full[n & 1]);
        if (it.mblk < 0) {
          finished = true;
          break;
        }
      }
      if (finished) {
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
          atomicExch(p.sched, 0);
          atomicExch(p.sched + 1, 0);
        }
      }
    }
  } else if (warp == kProducerWarp) {
    int G = 0, ni = 0;
    for (int n = 0;; ++n) {
      DqpItem it;
      bool ok = read_item(n, it);
      if (!__all_sync(0xffffffffu, ok)) break;
      __syncwarp();
      if (lane == 0) release_item(n);
      if (it.mblk < 0) break;
      const DqpWork w = dqp_decode(p, it);
      if (w.nb == 0) continue;
      if (lane == 0) {
        ok = mbar_wait(&xb->q_free, (ni & 1) ^ 1, ctx);
        if (ok) {
          mbar_arrive_expect_tx(&bars->fixed_full, 2 * C::kTileBytes + 1024);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c) {
            tma_load_4d(sQ + c * C::kChunkBytes, &p.tm_q, &bars->fixed_full, c * 64, w.head, w.q_off + w.row0, w.bq);
            tma_load_4d(sdO + c * C::kChunkBytes, &p.tm_do, &bars->fixed_full, c * 64, w.head, w.q_off + w.row0, w.bq);
          }
          const int64_t st = (static_cast<int64_t>(w.batch) * p.h + w.head) * p.sq_pad + w.row0;
          bulk_load_1d(sStats, p.lse2 + st, 512, &bars->fixed_full);
          bulk_load_1d(sStats + 128, p.delta + st, 512, &bars->fixed_full);
        }
        for (int j = 0; ok && j < w.nb; ++j) {
          const int g = G + j;
          const int s = g % C::kStagesK, sv = g % C::kStagesV;
          const int krow = w.k_off + j * kBlock;
          if (!(ok = mbar_wait(&bars->a_empty[s], ((g / C::kStagesK) & 1) ^ 1, ctx))) break;
          mbar_arrive_expect_tx(&bars->a_full[s], C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(sK + s * C::kTileBytes + c * C::kChunkBytes, &p.tm_k, &bars->a_full[s], c * 64, w.head_k, krow, w.bq);
          if (!(ok = mbar_wait(&bars->b_empty[sv], ((g / C::kStagesV) & 1) ^ 1, ctx))) break;
          mbar_arrive_expect_tx(&bars->b_full[sv], C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(sV + sv * C::kTileBytes + c * C::kChunkBytes, &p.tm_v, &bars->b_full[sv], c * 64, w.head_k, krow, w.bq);
        }
      }
      if (!__all_sync(0xffffffffu, ok)) break;
      if (w.fix_k_tail) {
        const int g = G + w.nkb - 1, s = g % C::kStagesK;
        if (!mbar_wait_warp(&bars->a_full[s], (g / C::kStagesK) & 1, ctx)) break;
        zero_tile_rows_from<D>(sK + s * C::kTileBytes, w.sk - (w.nkb - 1) * kBlock, lane);
        if (lane == 0) mbar_arrive(&bars->tail_fixed[0]);
      }
      G += w.nb;
      ++ni;
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_nn = make_idesc_f16(128, kBlock, false, false);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, ctx); };
      auto k_tile = [&](int g) { return smem_u32(sK + (g % C::kStagesK) * C::kTileBytes); };
      auto v_tile = [&](int g) { return smem_u32(sV + (g % C::kStagesV) * C::kTileBytes); };
      auto k_full = [&](int g) { return wait(&bars->a_full[g % C::kStagesK], (g / C::kStagesK) & 1); };
      auto v_full = [&](int g) { return wait(&bars->b_full[g % C::kStagesV], (g / C::kStagesV) & 1); };
      int G = 0, ni = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        DqpItem it;
        if (!(ok = read_item(n, it))) break;
        release_item(n);
        if (it.mblk < 0) break;
        const DqpWork w = dqp_decode(p, it);
        if (w.nb <= 2) mbar_arrive(&xb->sched_go);  // short item: claim the next one right away
        if (w.nb == 0) continue;
        ok = wait(&bars->fixed_full, ni & 1) && k_full(G);
        for (int j = 0; ok && j < w.nb; ++j) {
          const int g = G + j;
          if (g > 0 && !(ok = wait(&bars->s_loaded, (g - 1) & 1))) break;
          // S(g) complete tells the elementwise warps that packed-dS buffer g&1 is free again
          if (g >= 2 && !(ok = wait(&bars->ds_free[g & 1], ((g >> 1) - 1) & 1))) break;
          tc_fence_after_sync();
          ok = gemm_ss<D>(tmem_base + kColS, q_addr, k_tile(g), idesc_nn, [&] { return v_full(g); });
          if (!ok) break;
          tc_commit(&bars->s_full);
          tc_commit(&bars->a_empty[g % C::kStagesK]);  // second reader: the dQ MMAs of this block
          if (g > 0 && !(ok = wait(&bars->dp_loaded, (g - 1) & 1))) break;
          tc_fence_after_sync();
          ok = gemm_ss<D>(tmem_base + kColDP, do_addr, v_tile(g), idesc_nn,
                          [&] { return j + 1 >= w.nb || k_full(g + 1); });
          if (!ok) break;
          tc_commit(&bars->dp_full);
          tc_commit(&bars->b_empty[g % C::kStagesV]);
          if (j + 1 == w.nb) tc_commit(&xb->q_free);  // Q, dO and the statistics may be replaced
          if (w.nb > 2 && j + 3 == w.nb) mbar_arrive(&xb->sched_go);
        }
        G += w.nb;
        ++ni;
      }
    }
  } else if (warp == kAccMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, false, true);
      int G = 0, nf = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        DqpItem it;
        if (!(ok = read_item(n, it))) break;
        release_item(n);
        if (it.mblk < 0) break;
        const DqpWork w = dqp_decode(p, it);
        if (w.nb == 0) continue;
        for (int j = 0; ok && j < w.nb; ++j) {
          const int g = G + j, s = g % C::kStagesK;
          if (!(ok = mbar_wait(&bars->a_full[s], (g / C::kStagesK) & 1, ctx))) break;
          if (!(ok = mbar_wait(&bars->ds_full, g & 1, ctx))) break;
          if (w.fix_k_tail && j == w.nkb - 1 && !(ok = mbar_wait(&bars->tail_fixed[0], nf & 1, ctx))) break;
          tc_fence_after_sync();
          gemm_ts<D>(tmem_base + kColAcc, tmem_base + kColPacked + (g & 1) * 64, smem_u32(sK + s * C::kTileBytes),
                     idesc_acc, j == 0);
          tc_commit(&bars->a_empty[s]);
          tc_commit(&bars->ds_free[g & 1]);
        }
        if (ok) tc_commit(&bars->acc_full);
        G += w.nb;
        if (w.fix_k_tail) ++nf;
      }
    }
  } else if (warp < kComputeWarps) {
    // ---- elementwise warps: thread = (row, 32-column quarter) ----
    const int cq = warp >> 2, quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS + cq * 32;
    const uint32_t tDP = tmem_base + lane_base + kColDP + cq * 32;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    const bool varlen = p.cu_seqlens_q != nullptr;
    int G = 0, ni = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      int nb, sk, shift, row;
      {
        DqpItem it;
        ok = read_item(n, it);
        if (!(ok = __all_sync(0xffffffffu, ok))) break;
        if (it.mblk < 0) break;
        const DqpWork w = dqp_decode(p, it);
        nb = w.nb, sk = w.sk, shift = w.shift, row = w.row0 + row_in_tile;
      }
      float2 nl2 = make_float2(0.f, 0.f), nd2 = make_float2(0.f, 0.f);
      bool s_ready = false;
      for (int j = 0; j < nb; ++j) {
        const int g = G + j;
        if (!(ok = warp_wait_unless(s_ready, &bars->s_full, g & 1, ctx))) break;
        tc_fence_after_sync();
        uint32_t sr[32];
        tmem_ld32(tS, sr);
        const bool dp_ready = warp_probe(&bars->dp_full, g & 1);  // dP(j) follows S(j) through the pipe
        if (j == 0) {  // S(0) of the item was issued after its statistics had landed
          const float l = sStats[row_in_tile], dl = sStats[128 + row_in_tile];
          nl2 = make_float2(l, l), nd2 = make_float2(dl, dl);
        }
        tmem_wait_ld();
        warp_arrive_loaded(&bars->s_loaded, lane);
        const int col0 = j * kBlock + cq * 32;
        int limit = sk - 1 - col0;
        if (p.is_causal) limit = min(limit, row + shift - col0);
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
        if (!(ok = warp_wait_unless(dp_ready, &bars->dp_full, g & 1, ctx))) break;
        tc_fence_after_sync();
        tmem_ld32(tDP, sr);
        s_ready = j + 1 < nb && warp_probe(&bars->s_full, (g + 1) & 1);  // S(j+1) ran under the exponentials
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
        tmem_st16(tmem_base + lane_base + kColPacked + (g & 1) * 64 + cq * 16, pk);
        warp_arrive(&bars->ds_full, lane);
      }
      if (!ok) break;
      // ---- epilogue: dQ = scale * acc; what it needs of the item is derived again from the ring slot ----
      DqpItem it;
      {
        const volatile int* src = reinterpret_cast<const volatile int*>(&xb->items[n & 1]);
        it.batch = src[0], it.head = src[1], it.mblk = src[2], it.pad = 0;
      }
      const DqpWork w = dqp_decode(p, it);
      const bool stores = cq < D / 32;
      const int64_t dq_idx = (varlen ? static_cast<int64_t>(w.q_off + row) * p.dq_row_stride
                                     : w.batch * p.dq_batch_stride + static_cast<int64_t>(row) * p.dq_row_stride) +
                             w.head * p.dq_head_stride + cq * 32;
      if (nb > 0) {
        if (!(ok = mbar_wait_warp(&bars->acc_full, ni & 1, ctx))) break;
        ++ni;
      }
      if (stores) {
        if (nb > 0) {
          tc_fence_after_sync();
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_base + kColAcc + cq * 32, r);
          tmem_wait_ld();
          tc_fence_before_sync();
          if (row < w.sq) store_row_fp16(p.dq + dq_idx, r, p.scale);
        } else if (row < w.sq) {
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(p.dq + dq_idx + i * 8) = z;
        }
      }
      G += nb;
      __syncwarp();
      if (lane == 0) release_item(n);
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
// A work item is one 128-key tile of one (sequence, KV head): the CTA loops over the query heads of the GQA group
// and their Q tiles (iterations), S^T = K Q^T and dP^T = V dO^T per iteration (SS), P^T and dS^T in the elementwise
// warps, dV += P^T dO and dK += dS^T Q (TS) accumulated in TMEM over the whole group.  Persistent like the dQ
// kernel: one CTA per SM takes items from the work counter (heaviest causal key tile first), every barrier phase
// is derived from the cumulative iteration count T (or the item count), the K / V tiles of the next item are
// loaded as soon as the last dP^T product of the current item has read them, and its first S^T product is issued
// under the last elementwise iteration and the epilogue of the current one.  Dense batches only: packed (varlen)
// batches go to bwd_dkdv_packed_kernel below.
struct DkvItem {
  int batch, head_k, nblk, pad;  // nblk < 0: no more work
};
struct DkvBarriers {
  BBarriers b;
  uint64_t kv_free;         // the K / V tiles of the item have been read for the last time
  uint64_t sched_full[2], sched_empty[2], sched_go;
  DkvItem items[2];
};
static_assert(sizeof(DkvBarriers) <= 512, "barrier block");

struct DkvWork {
  int batch, head_k, sq, sk, key0, group, nq, i_min, shift, per_head, n_it;
};
__device__ __forceinline__ DkvWork dkv_decode(const BwdKernelParams& p, const DkvItem& it) {
  DkvWork w;
  w.batch = it.batch, w.head_k = it.head_k;
  w.sq = p.seqlen_q;
  w.sk = p.seqlen_k;
  w.key0 = it.nblk * kBlock;
  w.group = p.h / p.h_k;
  w.nq = (w.sq + kBlock - 1) / kBlock;
  w.i_min = 0;
  w.shift = (p.is_causal == 2) ? p.causal_shift : w.sk - w.sq;  // key j visible to query i iff j <= i + shift
  if (p.is_causal) {
    const int first_row = w.key0 - w.shift;  // first query row that can see key0
    w.i_min = first_row <= 0 ? 0 : first_row / kBlock;
  }
  w.per_head = max(0, w.nq - w.i_min);
  w.n_it = w.per_head * w.group;
  return w;
}

template <int D>
__global__ void __launch_bounds__(kDqpThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ BwdKernelParams p) {
  using C = BCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int stop_probe = stop_probe_begin(p.status);

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::kTileBytes;
  uint8_t* sQ = sV + C::kTileBytes;
  uint8_t* sdO = sQ + C::kStagesQ * C::kTileBytes;
  float* sStats = reinterpret_cast<float*>(sdO + C::kStagesDO * C::kTileBytes);  // [2][lse2 128 | delta 128]
  DkvBarriers* xb = reinterpret_cast<DkvBarriers*>(reinterpret_cast<uint8_t*>(sStats) + 2048);
  BBarriers* bars = &xb->b;
  if (smem - smem_raw > C::kAlignPadDkdv) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusSmemLayout);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == kProducerWarp && lane == 0) {
    init_barriers(bars, C::kStagesQ, 2, 2);
    mbar_init(&xb->kv_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&xb->sched_full[i], 1);
      mbar_init(&xb->sched_empty[i], kDqpReaders);
    }
    mbar_init(&xb->sched_go, 1);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  const bool stop = __syncthreads_or(stop_probe) != 0;  // sticky time-out bit set: the CTA does no work
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  WaitCtx ctx{&bars->abort_flag, p.status};

  auto read_item = [&](int n, DkvItem& it) -> bool {
    if (!mbar_wait(&xb->sched_full[n & 1], (n >> 1) & 1, ctx)) return false;
    it = xb->items[n & 1];
    return true;
  };
  auto release_item = [&](int n) { mbar_arrive(&xb->sched_empty[n & 1]); };

  if (stop) {
  } else if (warp == kDqpSchedWarp) {
    if (lane == 0) {
      bool finished = false;
      for (int n = 0;; ++n) {
        int next = blockIdx.x;
        if (n > 0) {
          if (!mbar_wait(&xb->sched_go, (n - 1) & 1, ctx)) break;
          next = gridDim.x + atomicAdd(p.sched, 1);
        }
        DkvItem it;
        it.batch = 0, it.head_k = 0, it.nblk = -1, it.pad = 0;
        if (next < p.total_items) {  // every index is a live item: key tile 0 of a head is the heaviest
          const int x = next % p.items_x, rest = next / p.items_x;
          it.head_k = rest % p.h_k, it.batch = rest / p.h_k, it.nblk = x;
        }
        if (!mbar_wait(&xb->sched_empty[n & 1], ((n >> 1) & 1) ^ 1, ctx)) break;
        xb->items[n & 1] = it;
        mbar_arrive(&xb->sched_full[n & 1]);
        if (it.nblk < 0) {
          finished = true;
          break;
        }
      }
      if (finished) {
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
          atomicExch(p.sched, 0);
          atomicExch(p.sched + 1, 0);
        }
      }
    }
  } else if (warp == kProducerWarp) {
    int T0 = 0, ni = 0;
    for (int n = 0;; ++n) {
      DkvItem item;
      bool ok = read_item(n, item);
      if (!__all_sync(0xffffffffu, ok)) break;
      __syncwarp();
      if (lane == 0) release_item(n);
      if (item.nblk < 0) break;
      const DkvWork w = dkv_decode(p, item);
      if (w.n_it == 0) continue;
      // Q tile, row statistics and dO tile of iteration `it` of the item into the rings at position T0 + it
      auto load_q_do = [&](int it) -> bool {
        const int T = T0 + it;
        const int sq_ = T % C::kStagesQ, sd = T % C::kStagesDO, ss = T & 1;
        const uint32_t phq = (T / C::kStagesQ) & 1, phd = (T / C::kStagesDO) & 1, phs = (T >> 1) & 1;
        const int head = w.head_k * w.group + it / w.per_head;
        const int i = w.i_min + it % w.per_head;
        const int qrow = i * kBlock;
        const int64_t stat = (static_cast<int64_t>(w.batch) * p.h + head) * p.sq_pad + i * kBlock;
        if (!mbar_wait(&bars->a_empty[sq_], phq ^ 1, ctx)) return false;
        mbar_arrive_expect_tx(&bars->a_full[sq_], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(sQ + sq_ * C::kTileBytes + c * C::kChunkBytes, &p.tm_q, &bars->a_full[sq_], c * 64, head, qrow, w.batch);
        if (!mbar_wait(&bars->st_empty[ss], phs ^ 1, ctx)) return false;
        mbar_arrive_expect_tx(&bars->st_full[ss], 1024);
        bulk_load_1d(sStats + ss * 256, p.lse2 + stat, 512, &bars->st_full[ss]);
        bulk_load_1d(sStats + ss * 256 + 128, p.delta + stat, 512, &bars->st_full[ss]);
        if (!mbar_wait(&bars->b_empty[sd], phd ^ 1, ctx)) return false;
        mbar_arrive_expect_tx(&bars->b_full[sd], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(sdO + sd * C::kTileBytes + c * C::kChunkBytes, &p.tm_do, &bars->b_full[sd], c * 64, head, qrow, w.batch);
        return true;
      };
      if (lane == 0) {
        ok = mbar_wait(&xb->kv_free, (ni & 1) ^ 1, ctx);
        if (ok) {
          mbar_arrive_expect_tx(&bars->fixed_full, 2 * C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c) {
            tma_load_4d(sK + c * C::kChunkBytes, &p.tm_k, &bars->fixed_full, c * 64, w.head_k, w.key0, w.batch);
            tma_load_4d(sV + c * C::kChunkBytes, &p.tm_v, &bars->fixed_full, c * 64, w.head_k, w.key0, w.batch);
          }
        }
      }
      if (lane == 0) {
        for (int it = 0; ok && it < w.n_it; ++it) ok = load_q_do(it);
      }
      if (!__all_sync(0xffffffffu, ok)) break;
      T0 += w.n_it;
      ++ni;
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_nn = make_idesc_f16(128, kBlock, false, false);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      // One accumulator region A holds S^T(T) and then dP^T(T): dP^T(T) is issued as soon as S^T(T)
      // sits in registers, S^T(T+1) as soon as dP^T(T) does.  The hooks wait for the TMA load the next
      // product reads.
      auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, ctx); };
      auto q_tile = [&](int T) { return smem_u32(sQ + (T % C::kStagesQ) * C::kTileBytes); };
      auto do_tile = [&](int T) { return smem_u32(sdO + (T % C::kStagesDO) * C::kTileBytes); };
      auto q_full = [&](int T) { return wait(&bars->a_full[T % C::kStagesQ], (T / C::kStagesQ) & 1); };
      auto do_full = [&](int T) { return wait(&bars->b_full[T % C::kStagesDO], (T / C::kStagesDO) & 1); };
      const uint32_t tA = tmem_base + kColS, tA2 = tmem_base + kColDPT<D>;
      constexpr bool kSharedRegion = kColDPT<D> == kColS;
      int T0 = 0, ni = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        DkvItem item;
        if (!(ok = read_item(n, item))) break;
        release_item(n);
        if (item.nblk < 0) break;
        const DkvWork w = dkv_decode(p, item);
        // the next item is claimed kGoAhead iterations before this one ends; a shorter item: right away
        constexpr int kGoAhead = 2;
        if (w.n_it <= kGoAhead) mbar_arrive(&xb->sched_go);
        if (w.n_it == 0) continue;
        ok = wait(&bars->fixed_full, ni & 1) && q_full(T0);
        for (int it = 0; ok && it < w.n_it; ++it) {
          const int T = T0 + it;
          // region A is free once its last content was read: dP^T(T-1) when the region is shared, S^T(T-1) otherwise
          if (T > 0 && !(ok = wait(kSharedRegion ? &bars->dp_loaded : &bars->s_loaded, (T - 1) & 1))) break;
          tc_fence_after_sync();
          ok = gemm_ss<D>(tA, k_addr, q_tile(T), idesc_nn, [&] { return do_full(T); });  // S^T = K Q^T
          if (!ok) break;
          tc_commit(&bars->s_full);
          tc_commit(&bars->a_empty[T % C::kStagesQ]);  // second reader: the dK MMAs of this tile
          // the region of dP^T is free once S^T(T) (shared) or dP^T(T-1) (own region) was read
          if (kSharedRegion) {
            if (!(ok = wait(&bars->s_loaded, T & 1))) break;
          } else if (T > 0) {
            if (!(ok = wait(&bars->dp_loaded, (T - 1) & 1))) break;
          }
          tc_fence_after_sync();
          ok = gemm_ss<D>(tA2, v_addr, do_tile(T), idesc_nn,  // dP^T = V dO^T
                          [&] { return it + 1 >= w.n_it || q_full(T + 1); });
          if (!ok) break;
          tc_commit(&bars->dp_full);
          tc_commit(&bars->b_empty[T % C::kStagesDO]);  // second reader: the dV MMAs of this tile
          if (it + 1 == w.n_it) tc_commit(&xb->kv_free);  // K and V may be replaced
          if (w.n_it > kGoAhead && it + kGoAhead + 1 == w.n_it) mbar_arrive(&xb->sched_go);
        }
        T0 += w.n_it;
        ++ni;
      }
    }
  } else if (warp == kAccMmaWarp) {
    if (lane == 0) {
      // dV += P^T dO as soon as the packed P^T is written, dK += dS^T Q likewise.
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, false, true);
      const uint32_t tP = tmem_base + kColDP, tDS = tmem_base + kColDP + 64;
      const uint32_t tDV = tmem_base + kColAcc, tDK = tmem_base + kColAcc + D;
      bool ok = true;
      int T0 = 0;
      for (int n = 0; ok; ++n) {
        DkvItem item;
        if (!(ok = read_item(n, item))) break;
        release_item(n);
        if (item.nblk < 0) break;
        const DkvWork w = dkv_decode(p, item);
        if (w.n_it == 0) continue;
        for (int it = 0; ok && it < w.n_it; ++it) {
          const int T = T0 + it;
          const int sq_ = T % C::kStagesQ, sd = T % C::kStagesDO;
          if (!(ok = mbar_wait(&bars->b_full[sd], (T / C::kStagesDO) & 1, ctx))) break;
          if (!(ok = mbar_wait(&bars->p_full, T & 1, ctx))) break;
          tc_fence_after_sync();
          gemm_ts<D>(tDV, tP, smem_u32(sdO + sd * C::kTileBytes), idesc_acc, it == 0);
          tc_commit(&bars->b_empty[sd]);
          tc_commit(&bars->p_free);
          if (!(ok = mbar_wait(&bars->a_full[sq_], (T / C::kStagesQ) & 1, ctx))) break;
          if (!(ok = mbar_wait(&bars->ds_full, T & 1, ctx))) break;
          tc_fence_after_sync();
          gemm_ts<D>(tDK, tDS, smem_u32(sQ + sq_ * C::kTileBytes), idesc_acc, it == 0);
          tc_commit(&bars->a_empty[sq_]);
          tc_commit(&bars->ds_free[0]);
        }
        if (ok) tc_commit(&bars->acc_full);
        T0 += w.n_it;
      }
    }
  } else if (warp < kComputeWarps) {
    // ---- elementwise warps: thread = (key row, 32-query-column quarter) ----
    const int cq = warp >> 2, quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tA = tmem_base + lane_base + kColS + cq * 32;         // S^T, then dP^T
    const uint32_t tP = tmem_base + lane_base + kColDP + cq * 16;        // packed P^T
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    const float* stats = sStats + cq * 32;
    int T0 = 0, ni = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      int n_it, per_head, cmin0;
      {
        DkvItem item;
        ok = read_item(n, item);
        if (!(ok = __all_sync(0xffffffffu, ok))) break;
        if (item.nblk < 0) break;
        const DkvWork w = dkv_decode(p, item);
        n_it = w.n_it, per_head = w.per_head;
        // causal: query column q of tile i is masked for this key when key > q + shift, i.e. the columns of
        // this thread's quarter below  key - shift - (i * 128 + cq * 32)  are masked
        cmin0 = p.is_causal ? (w.key0 + row_in_tile) - w.shift - (w.i_min * kBlock + cq * 32) : 0;
      }
      int i_rel = 0;  // Q tile within the current head
      for (int it = 0; it < n_it; ++it) {
        const int T = T0 + it;
        const int ss = T & 1;
        if (!(ok = mbar_wait_warp(&bars->st_full[ss], (T >> 1) & 1, ctx))) break;
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
        if (!(ok = mbar_wait_warp(&bars->s_full, T & 1, ctx))) break;
        tc_fence_after_sync();
        uint32_t sr[32];
        tmem_ld32(tA, sr);
        tmem_wait_ld();
        warp_arrive_loaded(&bars->s_loaded, lane);  // region A may now receive dP^T
        // columns below cmin are masked by causality (clamped to [0, 32])
        const int cmin = max(0, min(32, cmin0 - i_rel * kBlock));
        const bool col_masked = cmin != 0;
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
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            if (2 * e < cmin) pr[e].x = 0.f;
            if (2 * e + 1 < cmin) pr[e].y = 0.f;
          }
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack_half2(pr[e].x, pr[e].y);
        // the dV MMAs of the previous tile must have consumed the old P^T before it is overwritten
        if (T > 0 && !(ok = mbar_wait_warp(&bars->p_free, (T - 1) & 1, ctx))) break;
        tmem_st16(tP, pk);
        warp_arrive(&bars->p_full, lane);

        if (!(ok = mbar_wait_warp(&bars->dp_full, T & 1, ctx))) break;
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
        if (col_masked) {  // by selection, like P^T
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            if (2 * e < cmin) pk[e] &= 0xffff0000u;
            if (2 * e + 1 < cmin) pk[e] &= 0x0000ffffu;
          }
        }
        // the statistics of this tile are in use no longer
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->st_empty[ss]);
        if (T > 0 && !(ok = mbar_wait_warp(&bars->ds_free[0], (T - 1) & 1, ctx))) break;
        tmem_st16(tP + 64, pk);  // packed dS^T
        warp_arrive(&bars->ds_full, lane);
      }
      if (!ok) break;
      // ---- epilogue: column quarters 0,1 store the halves of dV, quarters 2,3 the halves of dK * scale; what it
      // needs of the item is derived again from the ring slot ----
      DkvItem item;
      {
        const volatile int* src = reinterpret_cast<const volatile int*>(&xb->items[n & 1]);
        item.batch = src[0], item.head_k = src[1], item.nblk = src[2], item.pad = 0;
      }
      const DkvWork w = dkv_decode(p, item);
      const int key = w.key0 + row_in_tile;
      const int which = cq >> 1;        // 0 = dV, 1 = dK
      const int col_half = cq & 1;      // which D/2 columns
      __half* dst_base = (which == 0) ? p.dv : p.dk;
      const int64_t bs = (which == 0) ? p.dv_batch_stride : p.dk_batch_stride;
      const int64_t rs = (which == 0) ? p.dv_row_stride : p.dk_row_stride;
      const int64_t hs = (which == 0) ? p.dv_head_stride : p.dk_head_stride;
      __half* dst = dst_base + w.batch * bs + static_cast<int64_t>(key) * rs + w.head_k * hs + col_half * (D / 2);
      const float mul = (which == 0) ? 1.f : p.scale;
      if (n_it > 0) {
        if (!(ok = mbar_wait_warp(&bars->acc_full, ni & 1, ctx))) break;
        ++ni;
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < D / 64; ++q) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_base + kColAcc + which * D + col_half * (D / 2) + q * 32, r);
          tmem_wait_ld();
          if (key < w.sk) store_row_fp16(dst + q * 32, r, mul);
        }
        tc_fence_before_sync();
      } else if (key < w.sk) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i3 = 0; i3 < D / 16; ++i3) *reinterpret_cast<uint4*>(dst + i3 * 8) = z;
      }
      T0 += n_it;
      __syncwarp();
      if (lane == 0) release_item(n);
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
// 4. dK/dV kernel for packed sequences, one CTA per (sequence, KV head, key tile)
// =============================================================================================
// The same products and hand-offs as bwd_dkdv_kernel, but launched as a grid of max_seqlen_k / 128 x h_k x b CTAs
// that each set up, process one key tile and exit.  Kept for packed (varlen) batches: there the persistent form
// was measured 8-16 % SLOWER (16 sequences of 256-4096 tokens, Hq32 Hkv8 D128; 8 % with equal lengths) although it
// is 3-11 % faster on dense batches of the same sizes, and the cause was not found in the time there was.
// A Q tile of a packed batch can hold rows of the neighbouring sequence; this kernel carries the code that guards
// against them (kVarlen is always true here).
template <int D, bool kVarlen>
__global__ void __launch_bounds__(kNumThreads, 1)
bwd_dkdv_packed_kernel(const __grid_constant__ BwdKernelParams p) {
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
  const int stop_probe = stop_probe_begin(p.status);
  const int bq = varlen ? 0 : batch;
  const int group = p.h / p.h_k;
  const int nq = (sq + kBlock - 1) / kBlock;
  int i_min = 0;
  const int shift = (p.is_causal == 2) ? p.causal_shift : sk - sq;  // key j visible to query i iff j <= i + shift
  if (p.is_causal) {
    const int first_row = key0 - shift;  // first query row that can see key0
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
  const bool stop = __syncthreads_or(stop_probe) != 0;  // sticky time-out bit set: the CTA does no work
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  if (stop && threadIdx.x == 0) bars->abort_flag = 1;  // the common exit then lets the loads issued above land

  // the last Q / dO tile of a packed sequence holds rows of the next sequence (see zero_tile_rows_from)
  const bool fix_q_tail = kVarlen && (sq % kBlock) != 0 && n_it > 0;
  const int q_tail_rows = sq - (nq - 1) * kBlock;  // valid rows of the last Q tile
  if (stop) {
  } else if (warp == kProducerWarp) {
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
    const int cmin0 = p.is_causal ? key - shift - (i_min * kBlock + cq * 32) : 0;
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
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesDkdv));
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dkdv_packed_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesDkdv));
    configured[dev & 63] = true;
  }
  if (stage_mask & 2) {
    static bool configured_p[64] = {};
    if (!configured_p[dev & 63]) {
      FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytesDq + 1024));
      configured_p[dev & 63] = true;
    }
    BwdKernelParams kq = kp;
    const int sms = device_sm_count();
    kq.sched = next_sched_slot();
    if (sms <= 0 || kq.sched == nullptr) return set_error(FA_ERR_CUDA, "fa_bwd: device attributes not available");
    kq.items_x = (p->seqlen_q + kBlock - 1) / kBlock;
    kq.b = p->b;
    const int64_t total = kq.cu_seqlens_q ? static_cast<int64_t>(p->h) * (p->total_q / kBlock + p->b)
                                          : static_cast<int64_t>(kq.items_x) * p->h * p->b;
    FA_CHECK_ARG(total < (1ll << 30), "fa_bwd: too many work items");
    kq.total_items = static_cast<int>(total);
    const int grid = kq.total_items < sms ? kq.total_items : sms;
    bwd_dq_kernel<D><<<grid, kDqpThreads, C::kSmemBytesDq + 1024, stream>>>(kq);
    FA_CHECK_CUDA(cudaGetLastError());
  }
  if (stage_mask & 4) {
    if (kp.cu_seqlens_q != nullptr) {  // packed sequences: one CTA per key tile (see bwd_dkdv_packed_kernel)
      dim3 grid_k((p->seqlen_k + kBlock - 1) / kBlock, p->h_k, p->b);
      bwd_dkdv_packed_kernel<D, true><<<grid_k, kNumThreads, C::kSmemBytesDkdv, stream>>>(kp);
    } else {
      BwdKernelParams kk = kp;
      const int sms = device_sm_count();
      kk.sched = next_sched_slot();
      if (sms <= 0 || kk.sched == nullptr) return set_error(FA_ERR_CUDA, "fa_bwd: device attributes not available");
      kk.items_x = (p->seqlen_k + kBlock - 1) / kBlock;
      kk.b = p->b;
      const int64_t total = static_cast<int64_t>(kk.items_x) * p->h_k * p->b;
      FA_CHECK_ARG(total < (1ll << 30), "fa_bwd: too many work items");
      kk.total_items = static_cast<int>(total);
      const int grid = kk.total_items < sms ? kk.total_items : sms;
      bwd_dkdv_kernel<D><<<grid, kDqpThreads, C::kSmemBytesDkdv, stream>>>(kk);
    }
    FA_CHECK_CUDA(cudaGetLastError());
  }
  return FA_OK;
}

}  // namespace
}  // namespace fa

namespace fa {
namespace {
// rows per head of the fp32 dQ accumulator of the single-kernel path (whole 128-row tiles per sequence)
int64_t dq_acc_rows(const FaBwdParams* p) {
  if (p->cu_seqlens_q != nullptr) return ((static_cast<int64_t>(p->total_q) + kBlock - 1) / kBlock + p->b) * kBlock;
  return static_cast<int64_t>(p->b) * round_up(p->seqlen_q, kBlock);
}
size_t stats_bytes(const FaBwdParams* p) { return (2 * stats_floats(p) * sizeof(float) + 255) / 256 * 256; }
}  // namespace
}  // namespace fa

extern "C" size_t fa_bwd_workspace_bytes(const FaBwdParams* p) {
  if (p == nullptr || p->b < 1 || p->h < 1 || p->seqlen_q < 1) return 0;
  if ((p->flags & FA_BWD_SINGLE_KERNEL) == 0) return 2 * fa::stats_floats(p) * sizeof(float);
  return fa::stats_bytes(p) + static_cast<size_t>(fa::dq_acc_rows(p)) * p->h * p->d * sizeof(float);
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
  FA_CHECK_ARG(p->is_causal >= 0 && p->is_causal <= 2, "fa_bwd: is_causal must be 0, 1 or FA_CAUSAL_SHIFT");
  FA_CHECK_ARG(p->is_causal != 2 || p->cu_seqlens_q == nullptr, "fa_bwd: FA_CAUSAL_SHIFT is for dense q / k / v only");
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
  FA_CHECK_ARG((reinterpret_cast<uintptr_t>(p->workspace) & 255) == 0, "fa_bwd: workspace must be 256-byte aligned");
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
  const bool fused = (p->flags & FA_BWD_SINGLE_KERNEL) != 0;
  float* dq_acc = fused ? reinterpret_cast<float*>(static_cast<uint8_t*>(p->workspace) + stats_bytes(p)) : nullptr;
  if (fused && (stage_mask & 1)) {
    // the accumulator starts at zero; the pairs of the single kernel add their dQ partials into it
    FA_CHECK_CUDA(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(dq_acc_rows(p)) * p->h * p->d * sizeof(float), stream));
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
  kp.causal_shift = p->causal_shift;
  kp.cu_seqlens_q = p->cu_seqlens_q;
  kp.cu_seqlens_k = p->cu_seqlens_k;
  kp.status = device_status_ptr();
  kp.dq_acc = dq_acc;
  kp.dq_acc_rows = fused ? dq_acc_rows(p) : 0;
  kp.total_q = p->total_q;
  kp.sched = nullptr;  // set per launch of the dQ kernel
  kp.items_x = 0;
  kp.total_items = 0;
  kp.b = p->b;
  if (fused) {
    if (stage_mask & 2) {
      rc = launch_bwd_fused(kp, p, stream);
      if (rc != FA_OK) return rc;
    }
    if (stage_mask & 4) return launch_bwd_dq_finalize(kp, p, stream);
    return FA_OK;
  }
  if (p->d == 128) return launch_bwd<128>(kp, p, stage_mask, stream);
  return launch_bwd<64>(kp, p, stage_mask, stream);
}
