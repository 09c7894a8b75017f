// KV-cache step for sm_100a: in-place append of the new tokens, split-KV attention of a few query
// rows against a contiguous or paged cache, and the log-sum-exp merge of the splits.
//
// The attend kernel is HBM-bound (every cached K and V byte is read exactly once per KV head; the
// query heads of a GQA group share the read), so it is built around the memory system:
//   * one CTA per (split, KV head, sequence); a producer warp streams 64-token K and V tiles with
//     TMA (16-byte aligned bulk copies, 128-byte swizzle, no multicast) through a ring of
//     mbarrier-guarded stages, pages looked up in block_table per tile;
//   * four consumer warps each take 16 tokens of every tile: S = Q K^T and O += P V run on
//     mma.sync.m16n8k16 with ldmatrix from the swizzled tiles -- the up to 16 (query position, head
//     of the group) rows form the M dimension, so the tensor work is negligible and no CUDA-core
//     dot products or shuffle reductions sit on the critical path;
//   * online softmax in registers with a lazily updated reference maximum; the four warps merge
//     their (m, l, O) through shared memory at the end.
// Algorithmic bytes per (sequence, KV head): 2 * L * D * 2 (K and V rows) + q/out rows.
//
// Replaces paged_append_kernel, kvcache_decode_split_kernel, kvcache_split_kernel and
// kvcache_split_kernel_legacy of the reference (csrc/flash_attn/src/kvcache_native.cu:148-871),
// the contiguous append loop of mha_fwd_kvcache (csrc/flash_attn/flash_api.cpp:643-654) and the
// split heuristic choose_num_splits (kvcache_native.cu:913-952).  Query blocks with more than 16
// (position, head) rows per KV head go to the tiled tcgen05 forward kernel instead (the reference
// routes them to its tiled kernel too, flash_api.cpp:668-714).
#include <algorithm>
#include <mutex>

#include "combine.h"
#include "fwd.h"
#define FA_WAIT_INLINE  // two waits in all: nothing to gain from the out-of-line form
#include "ptx.cuh"

namespace fa {
namespace {

constexpr int kTileTokens = 64;
constexpr int kConsumerWarps = 4;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxRows = 16;  // M of the mma: (query position, head in group) pairs

struct DecodeParams {
  CUtensorMap tm_k;
  CUtensorMap tm_v;
  const __half* q;
  __half* o;        // final output (num_splits == 1)
  float* lse;       // final LSE (num_splits == 1)
  float* o_accum;   // (splits, rows_total, D) partials (num_splits > 1)
  float* lse_accum; // (splits, rows_total)
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int seqlen_q, seqlen_new, h, h_k, group;
  int64_t rows_total;  // b * h * seqlen_q
  float scale_log2;
  int is_causal;
  const int* cache_seqlens;
  const int* cache_batch_idx;
  const int* block_table;
  int64_t block_table_batch_stride;
  int page_size;     // tokens per page (paged) or capacity per cache row (contiguous)
  int capacity;      // tokens a sequence can hold: max_blocks_per_seq * page_size, or the cache row length
  int num_splits;    // grid.x
  int chunk_tiles;   // > 0: split s owns tiles [s*chunk, (s+1)*chunk); 0: proportional ranges
  int* status;
};

template <int D>
struct DCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kTileTokens * 128;     // 64 tokens x 128 B
  static constexpr int kTileBytes = kChunks * kChunkBytes;  // one K or V tile
  static constexpr int kStages = (D == 128) ? 3 : 6;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kMergeBytes = kConsumerWarps * kMaxRows * (D + 2) * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*align*/;
  static_assert(kMergeBytes <= kStages * kStageBytes, "merge buffer aliases the stage ring");
};

struct DBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  int abort_flag;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of the 16-byte unit (token row r, 8-element column group c8) inside a swizzled tile.
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int r, int c8) {
  return (c8 >> 3) * DCfg<D>::kChunkBytes + r * 128 + (((c8 & 7) ^ (r & 7)) << 4);
}

template <int D>
__global__ void __launch_bounds__(kDecodeThreads, (D == 128) ? 2 : 2)
decode_kernel(const __grid_constant__ DecodeParams p) {
  using C = DCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const int split = blockIdx.x;
  const int head_k = blockIdx.y;
  const int batch = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rows = p.seqlen_q * p.group;  // valid rows of the 16-row M tile

  // ---- this CTA's token range ----
  // Lengths are clamped to the cache capacity on the device (the host does not have to read them back);
  // a clamp is reported through the status word.
  const int len_raw = p.cache_seqlens[batch] + p.seqlen_new;
  const int len = max(0, min(len_raw, p.capacity));
  if (len != len_raw && threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusCapacityClamped);
  const int n_tiles = (len + kTileTokens - 1) / kTileTokens;
  int tile_begin, tile_end;
  if (p.chunk_tiles > 0) {
    tile_begin = min(n_tiles, split * p.chunk_tiles);
    tile_end = min(n_tiles, tile_begin + p.chunk_tiles);
  } else {
    tile_begin = static_cast<int>(static_cast<int64_t>(n_tiles) * split / p.num_splits);
    tile_end = static_cast<int>(static_cast<int64_t>(n_tiles) * (split + 1) / p.num_splits);
  }
  const int my_tiles = tile_end - tile_begin;

  // row r of the M tile -> (query position, head); output row index in (b, h, seqlen_q) order
  auto out_row_index = [&](int r) -> int64_t {
    const int q_pos = r / p.group;
    const int head = head_k * p.group + (r - q_pos * p.group);
    return (static_cast<int64_t>(batch) * p.h + head) * p.seqlen_q + q_pos;
  };

  const bool stop = cta_should_stop(p.status);  // CTA-uniform
  if (my_tiles <= 0 || stop) {
    // empty split: neutral partial (or a zero row when there is nothing to attend to at all)
    for (int idx = threadIdx.x; idx < rows * (D / 2); idx += blockDim.x) {
      const int r = idx / (D / 2);
      const int c = (idx - r * (D / 2)) * 2;
      const int64_t orow = out_row_index(r);
      if (p.num_splits > 1) {
        float2* dst = reinterpret_cast<float2*>(p.o_accum + (split * p.rows_total + orow) * D + c);
        *dst = make_float2(0.f, 0.f);
      } else {
        const int q_pos = r / p.group;
        const int head = head_k * p.group + (r - q_pos * p.group);
        __half2* dst = reinterpret_cast<__half2*>(p.o + batch * p.o_batch_stride + q_pos * p.o_row_stride +
                                                  head * p.o_head_stride + c);
        *dst = __floats2half2_rn(0.f, 0.f);
      }
    }
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      const int64_t orow = out_row_index(r);
      if (p.num_splits > 1) p.lse_accum[split * p.rows_total + orow] = -INFINITY;
      else p.lse[orow] = 0.f;
    }
    return;
  }

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  DBarriers* bars = reinterpret_cast<DBarriers*>(smem + C::kStages * C::kStageBytes);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], kConsumerWarps);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx ctx{&bars->abort_flag, p.status};

  if (warp == kConsumerWarps) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      prefetch_tensormap(&p.tm_k);
      prefetch_tensormap(&p.tm_v);
      const int cache_row = p.cache_batch_idx ? p.cache_batch_idx[batch] : batch;
      for (int i = 0; i < my_tiles; ++i) {
        const int s = i % C::kStages;
        const uint32_t ph = (i / C::kStages) & 1;
        const int tok = (tile_begin + i) * kTileTokens;
        int row = tok, blk = cache_row;
        if (p.block_table) {
          blk = p.block_table[batch * p.block_table_batch_stride + tok / p.page_size];
          row = tok % p.page_size;
        }
        if (!mbar_wait(&bars->empty[s], ph ^ 1, ctx)) break;
        mbar_arrive_expect_tx(&bars->full[s], C::kStageBytes);
        uint8_t* dst = smem + s * C::kStageBytes;
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(dst + c * C::kChunkBytes, &p.tm_k, &bars->full[s], c * 64, head_k, row, blk);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_4d(dst + C::kTileBytes + c * C::kChunkBytes, &p.tm_v, &bars->full[s], c * 64,
                      head_k, row, blk);
      }
    }
  } else {
    // =========================== consumers ===========================
    const int g = lane >> 2;   // fragment row (and row + 8)
    const int t4 = lane & 3;   // fragment column pair
    // Q fragments (A operand, 16 x D), straight from global memory; rows >= `rows` are zero.
    uint32_t qa[D / 16][4];
    {
      auto q_ptr = [&](int r) -> const __half* {
        const int q_pos = r / p.group;
        const int head = head_k * p.group + (r - q_pos * p.group);
        return p.q + batch * p.q_batch_stride + q_pos * p.q_row_stride + head * p.q_head_stride;
      };
      const __half* r0p = g < rows ? q_ptr(g) : nullptr;
      const __half* r1p = (g + 8) < rows ? q_ptr(g + 8) : nullptr;
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const int c = k * 16 + t4 * 2;
        qa[k][0] = r0p ? *reinterpret_cast<const uint32_t*>(r0p + c) : 0u;
        qa[k][1] = r1p ? *reinterpret_cast<const uint32_t*>(r1p + c) : 0u;
        qa[k][2] = r0p ? *reinterpret_cast<const uint32_t*>(r0p + c + 8) : 0u;
        qa[k][3] = r1p ? *reinterpret_cast<const uint32_t*>(r1p + c + 8) : 0u;
      }
    }
    // causal limit per fragment row: key j visible iff j <= q_pos + len - seqlen_q
    int lim0 = len - 1, lim1 = len - 1;
    if (p.is_causal) {
      lim0 = min(lim0, g / p.group + len - p.seqlen_q);
      lim1 = min(lim1, (g + 8) / p.group + len - p.seqlen_q);
    }

    float oacc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY;  // reference maxima of rows g and g + 8 (raw score units)
    float l0 = 0.f, l1 = 0.f;              // per-thread partial row sums
    const float c = p.scale_log2;
    const int tok_in_tile = warp * 16;     // this warp's 16 tokens of every tile
    bool ok = true;

    for (int i = 0; i < my_tiles; ++i) {
      const int s = i % C::kStages;
      const uint32_t ph = (i / C::kStages) & 1;
      ok = mbar_wait(&bars->full[s], ph, ctx);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t sK = smem_u32(smem + s * C::kStageBytes);
      const uint32_t sV = sK + C::kTileBytes;
      const int tok0 = (tile_begin + i) * kTileTokens + tok_in_tile;  // first token of this warp

      if (tok0 < len) {
        // ---- S = Q K^T for 16 tokens: two n8 tiles ----
        float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3, rr = lane & 7;
          ldmatrix_x4(sK + tile_offset<D>(tok_in_tile + (mi >> 1) * 8 + rr, k * 2 + (mi & 1)), b0, b1,
                      b2, b3);
          mma_16816(sacc[0], qa[k], b0, b1);
          mma_16816(sacc[1], qa[k], b2, b3);
        }
        // ---- mask the tail / causal limit ----
        if (tok0 + 15 > min(lim0, lim1)) {
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const int col = tok0 + n * 8 + t4 * 2;
            if (col > lim0) sacc[n][0] = -INFINITY;
            if (col + 1 > lim0) sacc[n][1] = -INFINITY;
            if (col > lim1) sacc[n][2] = -INFINITY;
            if (col + 1 > lim1) sacc[n][3] = -INFINITY;
          }
        }
        // Rows of V past the end of the sequence may hold anything (uninitialised cache memory):
        // zero them so that 0 * garbage cannot produce NaN.  Only this warp reads these rows.
        // (warp-uniform condition)
        if (tok0 + 15 >= len) {
          for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
            const int r = idx / (D / 8), c8 = idx - r * (D / 8);
            if (tok0 + r >= len)
              *reinterpret_cast<uint4*>(smem + s * C::kStageBytes + C::kTileBytes +
                                        tile_offset<D>(tok_in_tile + r, c8)) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();  // order these generic writes before the next TMA refill
          __syncwarp();
        }
        // ---- online softmax with a lazy reference maximum ----
        float mx0 = fmaxf(fmaxf(sacc[0][0], sacc[0][1]), fmaxf(sacc[1][0], sacc[1][1]));
        float mx1 = fmaxf(fmaxf(sacc[0][2], sacc[0][3]), fmaxf(sacc[1][2], sacc[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        float a0 = 1.f, a1 = 1.f;
        bool need = false;
        if (mx0 > m0) {
          if (m0 == -INFINITY) m0 = mx0;
          else if ((mx0 - m0) * c > 8.f) { a0 = ex2f((m0 - mx0) * c); m0 = mx0; need = true; }
        }
        if (mx1 > m1) {
          if (m1 == -INFINITY) m1 = mx1;
          else if ((mx1 - m1) * c > 8.f) { a1 = ex2f((m1 - mx1) * c); m1 = mx1; need = true; }
        }
        if (__any_sync(0xffffffffu, need)) {
          l0 *= a0;
          l1 *= a1;
#pragma unroll
          for (int n = 0; n < D / 8; ++n) {
            oacc[n][0] *= a0; oacc[n][1] *= a0;
            oacc[n][2] *= a1; oacc[n][3] *= a1;
          }
        }
        const float nm0 = (m0 == -INFINITY) ? 0.f : -m0 * c;
        const float nm1 = (m1 == -INFINITY) ? 0.f : -m1 * c;
        uint32_t pa[4];
        {
          const float p00 = ex2f(fmaf(sacc[0][0], c, nm0)), p01 = ex2f(fmaf(sacc[0][1], c, nm0));
          const float p02 = ex2f(fmaf(sacc[0][2], c, nm1)), p03 = ex2f(fmaf(sacc[0][3], c, nm1));
          const float p10 = ex2f(fmaf(sacc[1][0], c, nm0)), p11 = ex2f(fmaf(sacc[1][1], c, nm0));
          const float p12 = ex2f(fmaf(sacc[1][2], c, nm1)), p13 = ex2f(fmaf(sacc[1][3], c, nm1));
          l0 += (p00 + p01) + (p10 + p11);
          l1 += (p02 + p03) + (p12 + p13);
          pa[0] = pack_half2(p00, p01);
          pa[1] = pack_half2(p02, p03);
          pa[2] = pack_half2(p10, p11);
          pa[3] = pack_half2(p12, p13);
        }
        // ---- O += P V ----
#pragma unroll
        for (int n = 0; n < D / 16; ++n) {
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3, rr = lane & 7;
          ldmatrix_x4_trans(sV + tile_offset<D>(tok_in_tile + (mi & 1) * 8 + rr, n * 2 + (mi >> 1)), b0,
                            b1, b2, b3);
          mma_16816(oacc[2 * n], pa, b0, b1);
          mma_16816(oacc[2 * n + 1], pa, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[s]);
    }

    // ---- merge the four warps: (m, l, O) through shared memory (aliases the stage ring) ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    named_barrier_sync(1, kConsumerWarps * 32);  // every warp is done reading the ring
    float* mbuf = reinterpret_cast<float*>(smem);
    // layout: [warp][row][D + 2] with the last two floats = (m, l)
    {
      float* w = mbuf + warp * kMaxRows * (D + 2);
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const int col = n * 8 + t4 * 2;
        *reinterpret_cast<float2*>(w + g * (D + 2) + col) = make_float2(oacc[n][0], oacc[n][1]);
        *reinterpret_cast<float2*>(w + (g + 8) * (D + 2) + col) = make_float2(oacc[n][2], oacc[n][3]);
      }
      if (t4 == 0) {
        w[g * (D + 2) + D] = m0;
        w[g * (D + 2) + D + 1] = l0;
        w[(g + 8) * (D + 2) + D] = m1;
        w[(g + 8) * (D + 2) + D + 1] = l1;
      }
    }
    named_barrier_sync(1, kConsumerWarps * 32);
    if (ok) {
      // 128 threads: thread -> (row, column slice)
      constexpr int kColsPerThread = D * kMaxRows / (kConsumerWarps * 32);  // 16 (D=128) or 8
      constexpr int kThreadsPerRow = D / kColsPerThread;                    // 8
      const int tid = threadIdx.x;
      const int r = tid / kThreadsPerRow;
      const int c0 = (tid - r * kThreadsPerRow) * kColsPerThread;
      if (r < rows) {
        float mw[kConsumerWarps], lw[kConsumerWarps];
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          mw[w] = mbuf[(w * kMaxRows + r) * (D + 2) + D];
          lw[w] = mbuf[(w * kMaxRows + r) * (D + 2) + D + 1];
          mt = fmaxf(mt, mw[w]);
        }
        float lt = 0.f, sc[kConsumerWarps];
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          sc[w] = (mw[w] == -INFINITY) ? 0.f : ex2f((mw[w] - mt) * c);
          lt += lw[w] * sc[w];
        }
        const bool dead = (mt == -INFINITY) || (lt == 0.f);
        const float inv = dead ? 0.f : 1.f / lt;
        float acc[kColsPerThread];
#pragma unroll
        for (int j = 0; j < kColsPerThread; ++j) acc[j] = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float* src = mbuf + (w * kMaxRows + r) * (D + 2) + c0;
#pragma unroll
          for (int j = 0; j < kColsPerThread; ++j) acc[j] = fmaf(src[j], sc[w], acc[j]);
        }
        const float lse_val = dead ? -INFINITY : (mt * c + __log2f(lt)) * kLn2;
        const int64_t orow = out_row_index(r);
        if (p.num_splits > 1) {
          float* dst = p.o_accum + (split * p.rows_total + orow) * D + c0;
#pragma unroll
          for (int j = 0; j < kColsPerThread; j += 4)
            *reinterpret_cast<float4*>(dst + j) =
                make_float4(acc[j] * inv, acc[j + 1] * inv, acc[j + 2] * inv, acc[j + 3] * inv);
          if (c0 == 0) p.lse_accum[split * p.rows_total + orow] = lse_val;
        } else {
          const int q_pos = r / p.group;
          const int head = head_k * p.group + (r - q_pos * p.group);
          __half* dst = p.o + batch * p.o_batch_stride + q_pos * p.o_row_stride + head * p.o_head_stride + c0;
#pragma unroll
          for (int j = 0; j < kColsPerThread; j += 8) {
            uint4 v;
            v.x = pack_half2(acc[j] * inv, acc[j + 1] * inv);
            v.y = pack_half2(acc[j + 2] * inv, acc[j + 3] * inv);
            v.z = pack_half2(acc[j + 4] * inv, acc[j + 5] * inv);
            v.w = pack_half2(acc[j + 6] * inv, acc[j + 7] * inv);
            *reinterpret_cast<uint4*>(dst + j) = v;
          }
          if (c0 == 0) p.lse[orow] = dead ? 0.f : lse_val;
        }
      }
    }
  }
  __syncthreads();
  if (bars->abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// append: k_new/v_new (b, s_new, h_k, d) -> cache rows / pages at cache_seqlens[b] + t
// ---------------------------------------------------------------------------------------------
struct AppendParams {
  __half* k_cache;
  __half* v_cache;
  const __half* k_new;
  const __half* v_new;
  int64_t kc_batch_stride, kc_row_stride, kc_head_stride;
  int64_t vc_batch_stride, vc_row_stride, vc_head_stride;
  int64_t kn_batch_stride, kn_row_stride, kn_head_stride;
  int64_t vn_batch_stride, vn_row_stride, vn_head_stride;
  int b, seqlen_new, h_k, d;
  int cache_batch, seqlen_cache;
  const int* cache_seqlens;
  const int* cache_batch_idx;
  const int* block_table;
  int64_t block_table_batch_stride;
  int max_blocks_per_seq;
};

__global__ void __launch_bounds__(256) append_kernel(const AppendParams p) {
  const int units_per_row = p.d / 8;  // 16-byte units per (token, head)
  const int64_t total = static_cast<int64_t>(p.b) * p.seqlen_new * p.h_k * units_per_row;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int u = static_cast<int>(idx % units_per_row);
    int64_t rest = idx / units_per_row;
    const int head = static_cast<int>(rest % p.h_k);
    rest /= p.h_k;
    const int t = static_cast<int>(rest % p.seqlen_new);
    const int batch = static_cast<int>(rest / p.seqlen_new);
    const int pos = p.cache_seqlens[batch] + t;
    int64_t blk, row;
    if (p.block_table) {
      const int slot = pos / p.seqlen_cache;
      if (pos < 0 || slot >= p.max_blocks_per_seq) continue;  // beyond capacity: never written
      blk = p.block_table[batch * p.block_table_batch_stride + slot];
      row = pos - slot * p.seqlen_cache;
    } else {
      if (pos < 0 || pos >= p.seqlen_cache) continue;
      blk = p.cache_batch_idx ? p.cache_batch_idx[batch] : batch;
      row = pos;
    }
    if (blk < 0 || blk >= p.cache_batch) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(p.k_new + batch * p.kn_batch_stride + t * p.kn_row_stride +
                                                     head * p.kn_head_stride + u * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(p.v_new + batch * p.vn_batch_stride + t * p.vn_row_stride +
                                                     head * p.vn_head_stride + u * 8);
    *reinterpret_cast<uint4*>(p.k_cache + blk * p.kc_batch_stride + row * p.kc_row_stride +
                              head * p.kc_head_stride + u * 8) = kv;
    *reinterpret_cast<uint4*>(p.v_cache + blk * p.vc_batch_stride + row * p.vc_row_stride +
                              head * p.vc_head_stride + u * 8) = vv;
  }
}

bool uses_decode_kernel(const FaKvcacheParams* p) {
  return static_cast<int64_t>(p->seqlen_q) * (p->h / p->h_k) <= kMaxRows;
}

int capacity_tokens(const FaKvcacheParams* p) {
  return p->block_table ? p->max_blocks_per_seq * p->seqlen_cache : p->seqlen_cache;
}

// Split plan.  An explicit request is honoured as given (proportional ranges per sequence).  With
// num_splits == 0 the lengths are unknown on the host (no synchronisation), so work is cut into
// fixed chunks of tiles instead: every CTA gets at most `chunk` tiles and the grid covers the cache
// capacity; CTAs past a sequence's end return at once.  The chunk is chosen so that the sequences at
// full capacity would give about four CTAs per SM-slot (2 resident CTAs x 148 SMs), with a floor of
// 8 tiles (512 tokens) so that the merge traffic stays small against the K/V bytes.
void plan_splits(const FaKvcacheParams* p, int* num_splits, int* chunk_tiles) {
  if (!uses_decode_kernel(p)) {
    *num_splits = 1;
    *chunk_tiles = 0;
    return;
  }
  if (p->num_splits > 0) {
    *num_splits = std::min(p->num_splits, 256);
    *chunk_tiles = 0;
    return;
  }
  const int cap_tiles = std::max(1, (capacity_tokens(p) + p->seqlen_new + kTileTokens - 1) / kTileTokens);
  const int64_t base_ctas = static_cast<int64_t>(p->b) * p->h_k;
  const int64_t target_ctas = 4 * 2 * 148;
  int64_t want = (target_ctas + base_ctas - 1) / base_ctas;  // splits per (sequence, KV head)
  want = std::max<int64_t>(1, std::min<int64_t>(want, 256));
  int chunk = static_cast<int>((cap_tiles + want - 1) / want);
  chunk = std::max(chunk, 8);
  int splits = (cap_tiles + chunk - 1) / chunk;
  if (splits <= 1) {
    *num_splits = 1;
    *chunk_tiles = 0;
  } else {
    *num_splits = splits;
    *chunk_tiles = chunk;
  }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <int D>
int launch_decode(const DecodeParams& dp, int b, int h_k, cudaStream_t stream) {
  using C = DCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FA_CHECK_CUDA(cudaFuncSetAttribute(decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       C::kSmemBytes));
    configured[dev & 63] = true;
  }
  dim3 grid(dp.num_splits, h_k, b);
  decode_kernel<D><<<grid, kDecodeThreads, C::kSmemBytes, stream>>>(dp);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

int validate(const FaKvcacheParams* p, const char* who) {
  FA_CHECK_ARG(p != nullptr, std::string(who) + ": params is NULL");
  if (p->d != 64 && p->d != 128)
    return set_error(FA_ERR_UNSUPPORTED, std::string(who) + ": head_dim must be 64 or 128");
  FA_CHECK_ARG(p->b >= 1 && p->seqlen_q >= 1 && p->h >= 1 && p->h_k >= 1 && p->h % p->h_k == 0,
               std::string(who) + ": bad b / seqlen_q / h / h_k");
  FA_CHECK_ARG(p->seqlen_new >= 0 && p->num_splits >= 0, std::string(who) + ": negative seqlen_new or num_splits");
  FA_CHECK_ARG(p->cache_batch >= 1 && p->seqlen_cache >= 1, std::string(who) + ": empty cache");
  if (p->block_table) {
    FA_CHECK_ARG(p->seqlen_cache % kTileTokens == 0, std::string(who) + ": page size must be a multiple of 64");
    FA_CHECK_ARG(p->cache_batch_idx == nullptr, std::string(who) + ": block_table excludes cache_batch_idx");
    FA_CHECK_ARG(p->max_blocks_per_seq >= 1, std::string(who) + ": max_blocks_per_seq must be positive");
  }
  return FA_OK;
}

}  // namespace
}  // namespace fa

extern "C" int fa_kvcache_num_splits(const FaKvcacheParams* p) {
  using namespace fa;
  int rc = validate(p, "fa_kvcache_num_splits");
  if (rc != FA_OK) return rc;
  int splits, chunk;
  plan_splits(p, &splits, &chunk);
  return splits;
}

extern "C" size_t fa_kvcache_workspace_bytes(const FaKvcacheParams* p) {
  using namespace fa;
  if (validate(p, "fa_kvcache_workspace_bytes") != FA_OK) return 0;
  int splits, chunk;
  plan_splits(p, &splits, &chunk);
  if (splits <= 1) return 0;
  const size_t rows = static_cast<size_t>(p->b) * p->h * p->seqlen_q;
  return align_up(static_cast<size_t>(splits) * rows * p->d * sizeof(float), 256) +
         align_up(static_cast<size_t>(splits) * rows * sizeof(float), 256);
}

extern "C" int fa_kvcache(const FaKvcacheParams* p, fa_stream_t stream_) {
  using namespace fa;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc = validate(p, "fa_kvcache");
  if (rc != FA_OK) return rc;
  FA_CHECK_ARG(p->q && p->k_cache && p->v_cache && p->o && p->lse && p->cache_seqlens,
               "fa_kvcache: q, k_cache, v_cache, o, lse, cache_seqlens must be non-NULL");
  FA_CHECK_ARG((p->k_new == nullptr) == (p->v_new == nullptr), "fa_kvcache: k_new and v_new go together");
  FA_CHECK_ARG(p->k_new != nullptr || p->seqlen_new == 0, "fa_kvcache: seqlen_new > 0 without k_new");
  FA_CHECK_ARG(aligned16(p->q) && aligned16(p->o) && p->q_row_stride % 8 == 0 && p->q_head_stride % 8 == 0 &&
                   p->q_batch_stride % 8 == 0 && p->o_row_stride % 8 == 0 && p->o_head_stride % 8 == 0 &&
                   p->o_batch_stride % 8 == 0,
               "fa_kvcache: q and o must be 16-byte aligned with strides that are multiples of 8 elements");
  rc = check_device_sm100();
  if (rc != FA_OK) return rc;

  // ---- 1. append ----
  if (p->k_new && p->seqlen_new > 0) {
    FA_CHECK_ARG(aligned16(p->k_new) && aligned16(p->v_new) && aligned16(p->k_cache) && aligned16(p->v_cache),
                 "fa_kvcache: k_new, v_new and the caches must be 16-byte aligned");
    const int64_t strides[] = {p->kc_batch_stride, p->kc_row_stride, p->kc_head_stride, p->vc_batch_stride,
                               p->vc_row_stride, p->vc_head_stride, p->kn_batch_stride, p->kn_row_stride,
                               p->kn_head_stride, p->vn_batch_stride, p->vn_row_stride, p->vn_head_stride};
    for (int64_t s : strides)
      FA_CHECK_ARG(s % 8 == 0, "fa_kvcache: cache and k_new/v_new strides must be multiples of 8 elements");
    AppendParams ap;
    ap.k_cache = static_cast<__half*>(p->k_cache);
    ap.v_cache = static_cast<__half*>(p->v_cache);
    ap.k_new = static_cast<const __half*>(p->k_new);
    ap.v_new = static_cast<const __half*>(p->v_new);
    ap.kc_batch_stride = p->kc_batch_stride; ap.kc_row_stride = p->kc_row_stride; ap.kc_head_stride = p->kc_head_stride;
    ap.vc_batch_stride = p->vc_batch_stride; ap.vc_row_stride = p->vc_row_stride; ap.vc_head_stride = p->vc_head_stride;
    ap.kn_batch_stride = p->kn_batch_stride; ap.kn_row_stride = p->kn_row_stride; ap.kn_head_stride = p->kn_head_stride;
    ap.vn_batch_stride = p->vn_batch_stride; ap.vn_row_stride = p->vn_row_stride; ap.vn_head_stride = p->vn_head_stride;
    ap.b = p->b; ap.seqlen_new = p->seqlen_new; ap.h_k = p->h_k; ap.d = p->d;
    ap.cache_batch = p->cache_batch; ap.seqlen_cache = p->seqlen_cache;
    ap.cache_seqlens = p->cache_seqlens; ap.cache_batch_idx = p->cache_batch_idx;
    ap.block_table = p->block_table; ap.block_table_batch_stride = p->block_table_batch_stride;
    ap.max_blocks_per_seq = p->max_blocks_per_seq;
    const int64_t total = static_cast<int64_t>(p->b) * p->seqlen_new * p->h_k * (p->d / 8);
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 8));
    append_kernel<<<blocks, 256, 0, stream>>>(ap);
    FA_CHECK_CUDA(cudaGetLastError());
  }

  // ---- 2. attend ----
  if (!uses_decode_kernel(p)) {
    // many query rows per KV head: tiled tcgen05 forward over the cache
    FaFwdParams f = {};
    f.q = p->q; f.k = p->k_cache; f.v = p->v_cache; f.o = p->o; f.lse = p->lse;
    f.q_batch_stride = p->q_batch_stride; f.q_row_stride = p->q_row_stride; f.q_head_stride = p->q_head_stride;
    f.k_batch_stride = p->kc_batch_stride; f.k_row_stride = p->kc_row_stride; f.k_head_stride = p->kc_head_stride;
    f.v_batch_stride = p->vc_batch_stride; f.v_row_stride = p->vc_row_stride; f.v_head_stride = p->vc_head_stride;
    f.o_batch_stride = p->o_batch_stride; f.o_row_stride = p->o_row_stride; f.o_head_stride = p->o_head_stride;
    f.lse_row_stride = p->seqlen_q;
    f.b = p->b; f.seqlen_q = p->seqlen_q; f.seqlen_k = p->seqlen_cache;
    f.h = p->h; f.h_k = p->h_k; f.d = p->d;
    f.k_batch = p->cache_batch;
    f.softmax_scale = p->softmax_scale; f.is_causal = p->is_causal;
    f.seqused_k = p->cache_seqlens;
    f.cache_batch_idx = p->cache_batch_idx;
    f.block_table = p->block_table;
    f.block_table_batch_stride = p->block_table_batch_stride;
    f.page_size = p->block_table ? p->seqlen_cache : 0;
    f.block_table_cols = p->block_table ? p->max_blocks_per_seq : 0;
    return run_fwd(&f, p->seqlen_new, stream);
  }

  int splits, chunk;
  plan_splits(p, &splits, &chunk);
  const int64_t rows_total = static_cast<int64_t>(p->b) * p->h * p->seqlen_q;
  DecodeParams dp;
  rc = make_tensor_map_4d(&dp.tm_k, p->k_cache, p->d, p->h_k, p->seqlen_cache, p->cache_batch,
                          p->kc_head_stride, p->kc_row_stride, p->kc_batch_stride, kTileTokens,
                          "fa_kvcache: k_cache");
  if (rc != FA_OK) return rc;
  rc = make_tensor_map_4d(&dp.tm_v, p->v_cache, p->d, p->h_k, p->seqlen_cache, p->cache_batch,
                          p->vc_head_stride, p->vc_row_stride, p->vc_batch_stride, kTileTokens,
                          "fa_kvcache: v_cache");
  if (rc != FA_OK) return rc;
  dp.q = static_cast<const __half*>(p->q);
  dp.o = static_cast<__half*>(p->o);
  dp.lse = p->lse;
  dp.o_accum = nullptr;
  dp.lse_accum = nullptr;
  if (splits > 1) {
    const size_t need = fa_kvcache_workspace_bytes(p);
    if (p->workspace == nullptr || p->workspace_bytes < need)
      return set_error(FA_ERR_WORKSPACE, "fa_kvcache: workspace smaller than fa_kvcache_workspace_bytes()");
    FA_CHECK_ARG(aligned16(p->workspace), "fa_kvcache: workspace must be 16-byte aligned");
    dp.o_accum = static_cast<float*>(p->workspace);
    dp.lse_accum = reinterpret_cast<float*>(
        static_cast<uint8_t*>(p->workspace) +
        align_up(static_cast<size_t>(splits) * rows_total * p->d * sizeof(float), 256));
  }
  dp.q_batch_stride = p->q_batch_stride; dp.q_row_stride = p->q_row_stride; dp.q_head_stride = p->q_head_stride;
  dp.o_batch_stride = p->o_batch_stride; dp.o_row_stride = p->o_row_stride; dp.o_head_stride = p->o_head_stride;
  dp.seqlen_q = p->seqlen_q; dp.seqlen_new = p->seqlen_new; dp.h = p->h; dp.h_k = p->h_k;
  dp.group = p->h / p->h_k;
  dp.rows_total = rows_total;
  dp.scale_log2 = p->softmax_scale * kLog2e;
  dp.is_causal = p->is_causal;
  dp.cache_seqlens = p->cache_seqlens;
  dp.cache_batch_idx = p->cache_batch_idx;
  dp.block_table = p->block_table;
  dp.block_table_batch_stride = p->block_table_batch_stride;
  dp.page_size = p->seqlen_cache;
  dp.capacity = capacity_tokens(p);
  dp.num_splits = splits;
  dp.chunk_tiles = chunk;
  dp.status = device_status_ptr();
  rc = (p->d == 128) ? launch_decode<128>(dp, p->b, p->h_k, stream) : launch_decode<64>(dp, p->b, p->h_k, stream);
  if (rc != FA_OK) return rc;

  // ---- 3. merge ----
  if (splits > 1)
    return launch_combine(dp.o_accum, dp.lse_accum, p->o, p->lse, rows_total, splits, p->h, p->seqlen_q, p->d,
                          p->o_batch_stride, p->o_row_stride, p->o_head_stride, stream);
  return FA_OK;
}

// ---------------------------------------------------------------------------------------------
// fa_kvcache_noalloc: the same KV-cache step for hosts that cannot allocate device memory.
//
// Who needs it: a serving loop whose device memory pool is frozen after start-up, a plugin that runs
// inside another runtime's callback or graph node where cudaMalloc is not allowed, a language binding
// that can launch but not allocate.  The split partials (O fp32, LSE) then live in the array below,
// which is part of the library image: every GPU that loads the library holds these 32 MiB until exit.
//
// `g_noalloc_scratch` is a device symbol.  In host code its name is only a host-side stand-in for the
// device array, not a device address, so it must never be passed to a kernel as it is; the device
// address is looked up once per device with cudaGetSymbolAddress (with that device current) and that
// pointer is what the kernels receive.
// ---------------------------------------------------------------------------------------------
namespace fa {
namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[FA_KVCACHE_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevicesNoAlloc = 64;
void* g_noalloc_ptr[kMaxDevicesNoAlloc] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device (set-up on the first call per device).
int noalloc_scratch_ptr(void** out) {
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevicesNoAlloc)
    return set_error(FA_ERR_UNSUPPORTED, "fa_kvcache_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    FA_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return set_error(FA_ERR_CUDA, "fa_kvcache_noalloc: scratch symbol has no device address");
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return FA_OK;
}

}  // namespace
}  // namespace fa

extern "C" int fa_kvcache_noalloc(const FaKvcacheParams* p, fa_stream_t stream) {
  using namespace fa;
  int rc = validate(p, "fa_kvcache_noalloc");
  if (rc != FA_OK) return rc;
  const size_t need = fa_kvcache_workspace_bytes(p);
  if (need > FA_KVCACHE_NOALLOC_SCRATCH_BYTES)
    return set_error(FA_ERR_WORKSPACE,
                     "fa_kvcache_noalloc: this call needs " + std::to_string(need) +
                         " bytes of split scratch, more than the built-in " +
                         std::to_string(static_cast<size_t>(FA_KVCACHE_NOALLOC_SCRATCH_BYTES)) +
                         " bytes; use fewer splits or fa_kvcache() with a caller-owned workspace");
  rc = check_device_sm100();
  if (rc != FA_OK) return rc;
  void* scratch = nullptr;
  rc = noalloc_scratch_ptr(&scratch);
  if (rc != FA_OK) return rc;
  FaKvcacheParams q = *p;
  q.workspace = scratch;
  q.workspace_bytes = FA_KVCACHE_NOALLOC_SCRATCH_BYTES;
  return fa_kvcache(&q, stream);
}
