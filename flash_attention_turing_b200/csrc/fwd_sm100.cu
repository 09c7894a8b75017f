// Forward attention for sm_100a: O = softmax(Q K^T * scale [+ causal]) V and LSE.
//
// A work item is 256 query rows of one (sequence, query head): two 128-row Q tiles that share every
// K/V block, so the tensor core always has the other tile's GEMMs to run while one tile is in its
// softmax.  The kernel is PERSISTENT: one CTA per SM takes items from a global counter (heaviest causal
// items of a head first, heads of a KV group next to each other, as a plain launch would order them) and
// keeps its barriers, TMEM allocation and K/V ring across items, so that the loads and the first products of
// the next item run under the tail and the epilogue of the current one.  Warp roles (352 threads):
//   warps 0-3   softmax of Q tile 0, ONE THREAD PER QUERY ROW (TMEM lane): the thread reads all 128 scores
//               of its row (32x32b loads), so maximum, sum, rescale decision and epilogue are thread-local
//   warps 4-7   softmax of Q tile 1
//   warp  8     TMA producer: the Q tiles of an item, then its K and V blocks through a ring of stages
//   warp  9     tcgen05.mma issuer (one thread); also owns the TMEM allocation
//   warp  10    scheduler (one thread): fetches item indices, skips items past the end of a packed
//               sequence and publishes the next live item through a two-entry ring in shared memory
// Eleven warps leave 168 registers per thread (three warps share one scheduler's register file), which is
// what lets a thread hold a whole row of scores.
// Both GEMMs run on tcgen05 with fp32 accumulators in TMEM:
//   S_t = Q_t K_j^T   A and B from shared memory (K-major, 128-byte swizzle as TMA writes them)
//   O_t += P_t V_j    A = P_t read from TMEM (fp16, aliased onto S_t), B = V_j from shared memory
//                     as an MN-major operand (V is stored keys x head_dim)
// TMEM columns: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [256+D,256+2D).
// The softmax keeps a lazily updated reference maximum: O and the row sum are rescaled only when
// the running maximum grew by more than 2^8 relative to the reference, which keeps P within fp16
// range and removes almost all rescale passes over O.
// All barrier phases are cumulative over the items of a CTA: every role counts the K/V blocks (ring position),
// the blocks of its tile (S / P hand-offs) and the items (Q, O, scheduler ring) it has seen.
//
// Replaces flash_fwd_kernel / compute_attn_1rowblock of the reference
// (csrc/flash_attn/src/flash_fwd_kernel.h:23-664) including its masking (src/mask.h:20-69), its
// varlen offsets (src/block_info.h:3-36) and its launch grid (src/flash_fwd_launch_template.h:60-75).
#include "fwd.h"

#include "ptx.cuh"

namespace fa {

namespace {

constexpr int kBlockM = 128;   // rows per Q tile
constexpr int kTiles = 2;      // Q tiles per work item
constexpr int kBlockN = 128;   // keys per K/V block
constexpr int kNumThreads = 352;
constexpr int kSoftmaxWarpsPerTile = 4;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kSchedWarp = 10;
constexpr int kSchedDepth = 2;
constexpr int kSchedReaders = kTiles * kSoftmaxWarpsPerTile + 2;  // softmax warps, producer warp, MMA thread
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdKernelParams {
  CUtensorMap tm_q;
  CUtensorMap tm_k;
  CUtensorMap tm_v;
  __half* o;
  float* lse;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t lse_row_stride;
  int seqlen_q, seqlen_k;
  int h, h_k;
  float scale;       // softmax scale
  float scale_log2;  // softmax scale * log2(e)
  int is_causal;
  int causal_shift;   // is_causal == 2: key j visible to query i iff j <= i + causal_shift (else sk - sq is used)
  const int* cu_seqlens_q;
  const int* cu_seqlens_k;
  const int* seqused_k;
  int seqused_k_add;  // added to seqused_k[b] (tokens appended to a cache in the same call)
  int k_capacity;     // upper bound for seqused_k: rows of k, or block_table columns * page_size
  const int* cache_batch_idx;
  const int* block_table;
  int64_t block_table_batch_stride;
  int page_size;
  int* status;
  int* sched;         // {next item - gridDim.x, CTAs finished}: both zero at launch and again at the end
  int items_x;        // dense: work items per (sequence, head) = ceil(seqlen_q / 256)
  int total_items;    // dense: items_x * h * b; packed sequences: h * (total_q / 256 + b), see the scheduler
  int b;              // sequences
};

template <int D>
struct Cfg {
  static constexpr int kChunks = D / 64;              // 128-byte swizzle chunks per row
  static constexpr int kChunkBytes = 128 * 128;       // 128 rows x 128 B
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kColS = 0;                     // + 128 * tile
  static constexpr int kColO = 256;                   // + D * tile
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes =
      kTiles * kTileBytes + 2 * kStages * kTileBytes + 1024 /*barriers*/ + 1024 /*alignment*/;
};

struct WorkItem {
  int batch, head, mpair;  // mpair: index of the 256-row pair of Q tiles; < 0: no more work
  int pad;
};

struct Barriers {
  uint64_t q_full, q_empty;    // both Q tiles of an item loaded / read by the last S MMA of the item
  uint64_t s_full[kTiles];
  uint64_t p_full[kTiles][2];  // P chunk c (key slices {2c, 2c+1} of each 64-key half) written
  uint64_t o_full[kTiles];
  uint64_t k_full[4];
  uint64_t k_empty[4];
  uint64_t v_full[4];
  uint64_t v_empty[4];
  uint64_t v_fixed;         // rows of the last V block past the sequence end have been zeroed
  uint64_t sched_full[kSchedDepth];
  uint64_t sched_empty[kSchedDepth];
  uint64_t sched_go;        // the current item is two blocks from its end: time to claim the next one
  WorkItem items[kSchedDepth];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= 1024, "barrier block");

// eleven warps: three on one SM sub-partition (16384 registers): 3 x 32 x 168 fits; a budget that does not fit
// cannot be scheduled at all
static_assert((kNumThreads / 32 + 3) / 4 * 32 * 168 <= 16384, "register file of one SM sub-partition");

// What every role derives from a work item.
struct Work {
  int batch, head, head_k, bq, bk;
  int q_off, k_off, sq, sk;
  int row0, shift, nkb;
  int nb[kTiles], nb_max;
  bool fix_v_tail;
};

__device__ __forceinline__ Work decode_work(const FwdKernelParams& p, const WorkItem& it) {
  Work w;
  w.batch = it.batch;
  w.head = it.head;
  const bool varlen_q = p.cu_seqlens_q != nullptr;
  const bool varlen_k = p.cu_seqlens_k != nullptr;
  w.q_off = varlen_q ? p.cu_seqlens_q[w.batch] : 0;
  w.sq = varlen_q ? p.cu_seqlens_q[w.batch + 1] - w.q_off : p.seqlen_q;
  w.k_off = varlen_k ? p.cu_seqlens_k[w.batch] : 0;
  w.sk = varlen_k ? p.cu_seqlens_k[w.batch + 1] - w.k_off : p.seqlen_k;
  if (p.seqused_k) {
    // clamped to what the K/V tensor (or the block table) can hold; the scheduler thread reports a clamp
    w.sk = max(0, min(p.seqused_k[w.batch] + p.seqused_k_add, p.k_capacity));
  }
  w.row0 = it.mpair * (kTiles * kBlockM);
  w.bq = varlen_q ? 0 : w.batch;
  w.bk = varlen_k ? 0 : (p.cache_batch_idx ? p.cache_batch_idx[w.batch] : w.batch);
  w.head_k = w.head / (p.h / p.h_k);
  // causal diagonal: key j is visible to query i iff j <= i + shift
  w.shift = (p.is_causal == 2) ? p.causal_shift : w.sk - w.sq;
  // number of K/V blocks each tile visits
  w.nkb = (w.sk + kBlockN - 1) / kBlockN;
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int r0 = w.row0 + t * kBlockM;
    int n = w.nkb;
    if (p.is_causal) {
      const int x = r0 + kBlockM + w.shift;  // one past the last visible key of the tile's last row
      n = x <= 0 ? 0 : min(w.nkb, (x + kBlockN - 1) / kBlockN);
    }
    if (r0 >= w.sq) n = 0;
    w.nb[t] = n;
  }
  w.nb_max = max(w.nb[0], w.nb[1]);
  // Rows of the last K/V block that lie past the end of the sequence are real memory when the keys come
  // from a packed tensor or a cache (the next sequence, or never-written cache rows).  Their scores are
  // masked, but P = 0 times a NaN/Inf bit pattern in V would still poison O, so those V rows are zeroed
  // in shared memory before the last PV MMA.  (Dense tensors: TMA fills out-of-range rows with zeros.)
  w.fix_v_tail = (p.seqused_k != nullptr || varlen_k) && (w.sk % kBlockN) != 0 && w.nb_max == w.nkb && w.nkb > 0;
  return w;
}

template <int D>
__global__ void __maxnreg__(168)
fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];

  if (cta_should_stop(p.status)) return;

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle) ----
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTiles * C::kTileBytes;
  uint8_t* sV = sK + C::kStages * C::kTileBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(sV + C::kStages * C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;


  if (warp == kProducerWarp && lane == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 1);
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_full[t][0], kSoftmaxWarpsPerTile);
      mbar_init(&bars->p_full[t][1], kSoftmaxWarpsPerTile);
      mbar_init(&bars->o_full[t], 1);
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->v_fixed, 1);
    for (int s = 0; s < kSchedDepth; ++s) {
      mbar_init(&bars->sched_full[s], 1);
      mbar_init(&bars->sched_empty[s], kSchedReaders);
    }
    mbar_init(&bars->sched_go, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  // Item n of this CTA, read by a whole warp (or by a single thread); false when the CTA is aborting.
  // tag of the waiting role in the status word: 1 softmax, 2 producer, 3 MMA issuer, 4 scheduler
  auto read_item = [&](int n, WorkItem& it, const WaitCtx& ctx) -> bool {
    const int slot = n % kSchedDepth;
    if (!mbar_wait(&bars->sched_full[slot], (n / kSchedDepth) & 1, ctx)) return false;
    it = bars->items[slot];
    return true;
  };
  auto release_item = [&](int n) { mbar_arrive(&bars->sched_empty[n % kSchedDepth]); };

  if (warp == kSchedWarp) {
    // =========================== scheduler ===========================
    const WaitCtx ctx{&bars->abort_flag, p.status, 4, bars};
    if (lane == 0) {
      // An item is claimed only when the previous one is two blocks from its end (the MMA thread says when):
      // early enough for its Q tiles and first K/V blocks to arrive in time, late enough that no CTA sits on
      // claimed work while another runs dry at the end of the launch (claiming one or two items ahead cost
      // 7 % at sequence length 65536).
      bool finished = false;
      int seq = 0;  // packed sequences: the sequence of the last claimed index
      for (int n = 0;; ++n) {
        const int slot = n % kSchedDepth;
        int next = blockIdx.x;  // the first item of a CTA needs no counter
        if (n > 0) {
          if (!mbar_wait(&bars->sched_go, (n - 1) & 1, ctx)) break;
          next = gridDim.x + atomicAdd(p.sched, 1);
        }
        WorkItem it;
        it.batch = 0, it.head = 0, it.mpair = -1, it.pad = 0;
        while (next < p.total_items) {
          int batch, head, mpair;
          if (p.cu_seqlens_q == nullptr) {
            const int x = next % p.items_x, rest = next / p.items_x;
            head = rest % p.h, batch = rest / p.h;
            mpair = p.items_x - 1 - x;  // heavy (late-row) causal items of a head first
          } else {
            // Packed sequences: sequence k owns the slots [h * v(k), h * v(k+1)) with v(k) = cu_seqlens_q[k] / 256 + k,
            // which are at least h * ceil(length / 256) and at most h more -- so an index maps to a live item
            // except for at most one slot per (sequence, head), whatever the spread of the lengths.  The indices
            // a CTA claims only grow, so the sequence is found by walking forward from the last one.
            while (seq + 1 < p.b && p.h * ((p.cu_seqlens_q[seq + 1] >> 8) + seq + 1) <= next) ++seq;
            const int v0 = (p.cu_seqlens_q[seq] >> 8) + seq, v1 = (p.cu_seqlens_q[seq + 1] >> 8) + seq + 1;
            const int rel = next - p.h * v0, cnt = v1 - v0;
            const int len = p.cu_seqlens_q[seq + 1] - p.cu_seqlens_q[seq];
            batch = seq, head = rel / cnt;
            mpair = (len + kTiles * kBlockM - 1) / (kTiles * kBlockM) - 1 - rel % cnt;  // < 0: the spare slot
            if (head >= p.h) mpair = -1;  // past the last sequence
          }
          const int sq = p.cu_seqlens_q ? p.cu_seqlens_q[batch + 1] - p.cu_seqlens_q[batch] : p.seqlen_q;
          if (mpair >= 0 && mpair * (kTiles * kBlockM) < sq) {
            it.batch = batch, it.head = head, it.mpair = mpair;
            if (p.seqused_k && p.status && head == 0 && mpair == 0) {
              const int raw = p.seqused_k[batch] + p.seqused_k_add;
              if (raw < 0 || raw > p.k_capacity) atomicOr(p.status, kStatusCapacityClamped);
            }
            break;
          }
          next = gridDim.x + atomicAdd(p.sched, 1);  // a spare slot: skip
        }
        if (!mbar_wait(&bars->sched_empty[slot], ((n / kSchedDepth) & 1) ^ 1, ctx)) break;
        bars->items[slot] = it;
        mbar_arrive(&bars->sched_full[slot]);
        if (it.mpair < 0) {
          finished = true;
          break;
        }
      }
      if (finished) {
        // the last CTA to run out of work puts the counters back to zero for the launch that takes them next
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
          atomicExch(p.sched, 0);
          atomicExch(p.sched + 1, 0);
        }
      }
    }
  } else if (warp == kProducerWarp) {
    // =========================== TMA producer ===========================
    const WaitCtx ctx{&bars->abort_flag, p.status, 2, bars};
    int g = 0;   // K/V blocks loaded so far: ring position
    int nq = 0;  // items whose Q tiles were loaded
    for (int n = 0;; ++n) {
      WorkItem it;
      bool ok = read_item(n, it, ctx);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      __syncwarp();
      if (lane == 0) release_item(n);
      if (it.mpair < 0) break;
      const Work w = decode_work(p, it);
      if (w.nb_max == 0) continue;
      if (lane == 0) {
        ok = mbar_wait(&bars->q_empty, (nq & 1) ^ 1, ctx);
        if (ok) {
          const int ntl = (w.nb[0] > 0) + (w.nb[1] > 0);
          mbar_arrive_expect_tx(&bars->q_full, ntl * C::kTileBytes);
#pragma unroll
          for (int t = 0; t < kTiles; ++t) {
            if (w.nb[t] > 0) {
#pragma unroll
              for (int c = 0; c < C::kChunks; ++c)
                tma_load_4d(sQ + t * C::kTileBytes + c * C::kChunkBytes, &p.tm_q, &bars->q_full, c * 64, w.head,
                            w.q_off + w.row0 + t * kBlockM, w.bq);
            }
          }
        }
        for (int j = 0; ok && j < w.nb_max; ++j) {
          const int gj = g + j;
          const int s = gj % C::kStages;
          const uint32_t ph = (gj / C::kStages) & 1;
          int krow = w.k_off + j * kBlockN;
          int kb = w.bk;
          if (p.block_table) {
            const int tok = j * kBlockN;
            kb = p.block_table[w.batch * p.block_table_batch_stride + tok / p.page_size];
            krow = tok % p.page_size;
          }
          if (!(ok = mbar_wait(&bars->k_empty[s], ph ^ 1, ctx))) break;
          mbar_arrive_expect_tx(&bars->k_full[s], C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(sK + s * C::kTileBytes + c * C::kChunkBytes, &p.tm_k, &bars->k_full[s], c * 64, w.head_k,
                        krow, kb);
          if (!(ok = mbar_wait(&bars->v_empty[s], ph ^ 1, ctx))) break;
          mbar_arrive_expect_tx(&bars->v_full[s], C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            tma_load_4d(sV + s * C::kTileBytes + c * C::kChunkBytes, &p.tm_v, &bars->v_full[s], c * 64, w.head_k,
                        krow, kb);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (w.fix_v_tail) {
        const int gj = g + w.nkb - 1;
        const int s = gj % C::kStages;
        if (!mbar_wait_warp(&bars->v_full[s], (gj / C::kStages) & 1, ctx)) break;
        // zero whole 128-byte row segments: the swizzle only permutes 16-byte units inside a row
        const int first = w.sk - (w.nkb - 1) * kBlockN;  // first invalid row of the block
        uint8_t* tile = sV + s * C::kTileBytes;
        for (int idx = lane; idx < (kBlockN - first) * C::kChunks * 8; idx += 32) {
          const int r = first + idx / (C::kChunks * 8);
          const int u = idx % (C::kChunks * 8);
          *reinterpret_cast<uint4*>(tile + (u >> 3) * C::kChunkBytes + r * 128 + (u & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->v_fixed);
      }
      g += w.nb_max;
      ++nq;
    }
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    const WaitCtx ctx{&bars->abort_flag, p.status, 3, bars};
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(128, kBlockN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, D, false, true);
      const uint32_t sQ_addr = smem_u32(sQ);
      const uint32_t sK_addr = smem_u32(sK);
      const uint32_t sV_addr = smem_u32(sV);

      // The products are written ONCE each, with the tile index as a run-time value and the first S products of
      // an item folded into the block loop (step j = -1): all warp roles execute different code at the same
      // time and the kernel runs close to the capacity of the instruction cache, so code size is throughput.
      // S_t = Q_t K^T with K in ring stage s: D/16 MMAs of K=16; slice k lives in swizzle chunk k/4 at byte
      // (k%4)*32.
      auto issue_qk = [&](int t, int s) {
        const uint64_t qd = make_smem_desc(sQ_addr + t * C::kTileBytes, 16, 1024);
        const uint64_t kd = make_smem_desc(sK_addr + s * C::kTileBytes, 16, 1024);
        const uint32_t d_addr = tmem_base + C::kColS + t * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * C::kChunkBytes + (k & 3) * 32;
          mma_ss(d_addr, desc_advance(qd, off), desc_advance(kd, off), idesc_qk, k > 0);
        }
      };
      // O_t += P_t V in two steps: chunk c = keys [64c, 64c+64) = K=16 slices 4c..4c+3.  A slice k = 8
      // TMEM columns of packed fp16 at the start of the S_t region; B slice k starts 16 key rows (2048 B)
      // further, head_dim chunks are kChunkBytes apart (LBO).  The softmax warps hand over P in two steps so
      // that the first half of the PV MMAs runs under the exponentials of the second.
      auto issue_pv = [&](int t, int s, int c, bool first_block) {
        const uint64_t vd = make_smem_desc(sV_addr + s * C::kTileBytes + c * 4 * 2048, C::kChunkBytes, 1024);
        const uint32_t d_addr = tmem_base + C::kColO + t * D;
        const uint32_t a_addr = tmem_base + C::kColS + t * 128 + c * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          mma_ts(d_addr, a_addr + i * 8, desc_advance(vd, i * 2048), idesc_pv, (!first_block || c > 0 || i > 0) ? 1u : 0u);
      };

      int g = 0;            // K/V blocks consumed so far: ring position
      int nq = 0;           // items with Q tiles
      int nf = 0;           // items whose last V block had to be fixed
      uint32_t cs_par = 0;  // bit t: parity of the number of blocks tile t has had: phase of its P hand-offs
      bool ok = true;
#pragma unroll 1
      for (int n = 0; ok; ++n) {
        WorkItem it;
        if (!(ok = read_item(n, it, ctx))) break;
        release_item(n);
        if (it.mpair < 0) break;
        const Work w = decode_work(p, it);
        const int nb0 = w.nb[0], nb1 = w.nb[1], nb_max = w.nb_max;
        if (nb_max <= 2) mbar_arrive(&bars->sched_go);  // short item: claim the next one right away
        if (nb_max == 0) continue;
        if (!(ok = mbar_wait(&bars->q_full, nq & 1, ctx))) break;
        if (!(ok = mbar_wait(&bars->k_full[g % C::kStages], (g / C::kStages) & 1, ctx))) break;
        tc_fence_after_sync();
        // step j: O_t += P_t(j) V(j), then S_t(j+1) = Q_t K(j+1)^T; step -1 issues only S_t(0)
#pragma unroll 1
        for (int j = -1; ok && j < nb_max; ++j) {
          const int s = (g + j) % C::kStages;  // unused at j = -1
          const int s1 = (g + j + 1) % C::kStages;
          // V(j) and K(j+1) are not polled here: a barrier poll costs this thread 60-130 clocks in which it
          // issues nothing, so the softmax warps observe v_full / k_full while they wait for S anyway, and
          // their p_full arrival carries the observation over (mbarrier release/acquire is cumulative).
          if (w.fix_v_tail && j == w.nkb - 1 && !(ok = mbar_wait(&bars->v_fixed, nf & 1, ctx))) break;
#pragma unroll
          for (int t = 0; t < kTiles; ++t) {
            const int nbt = t ? nb1 : nb0;
            const bool has_pv = j >= 0 && j < nbt;
            if (has_pv) {
              const uint32_t par = (cs_par >> t) & 1;
              if (!(ok = mbar_wait_hot(&bars->p_full[t][0], par, ctx))) break;
              tc_fence_after_sync();
              issue_pv(t, s, 0, j == 0);
              if (!(ok = mbar_wait_hot(&bars->p_full[t][1], par, ctx))) break;
              tc_fence_after_sync();
              issue_pv(t, s, 1, j == 0);
              cs_par ^= 1u << t;
              if (t == kTiles - 1 || !(j < nb1)) tc_commit(&bars->v_empty[s]);  // last reader of V(j)
            }
            if (j + 1 < nbt) {
              issue_qk(t, s1);
              tc_commit(&bars->s_full[t]);
              if (t == kTiles - 1 || !(j + 1 < nb1)) {  // last reader of K(j+1)
                tc_commit(&bars->k_empty[s1]);
                if (j + 2 == nb_max) tc_commit(&bars->q_empty);  // the last S MMAs of the item are issued
                if (nb_max > 2 && j + 3 == nb_max) mbar_arrive(&bars->sched_go);
              }
            } else if (has_pv) {
              tc_commit(&bars->o_full[t]);
            }
          }
        }
        g += nb_max;
        ++nq;
        if (w.fix_v_tail) ++nf;
      }
    }
  } else {
    // =========================== softmax + epilogue ===========================
    // One thread per query row (TMEM lane): warps 0-3 own Q tile 0, warps 4-7 Q tile 1, and thread `lane`
    // of warp w owns row 32 * (w % 4) + lane of its tile with all 128 score columns of a block (32x32b TMEM
    // loads).  Row maximum, row sum, rescale decision and the epilogue are thread-local: no shuffles, no
    // exchange between warps.  With eleven warps per CTA a thread may use 168 registers, enough to hold 128
    // scores at once, so the maximum needs one round of loads; only columns 64-127 are read a second time
    // (the packed P overwrites columns 0-63 of the S region, which are kept in registers).
    const WaitCtx ctx{&bars->abort_flag, p.status, 1, bars};
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + C::kColS + t * 128;
    const uint32_t tO = tmem_base + lane_base + C::kColO + t * D;
    const float c = p.scale_log2;
    const bool varlen_q = p.cu_seqlens_q != nullptr;

    auto hand_over = [&](int chunk) {  // all lanes have written their share of the P chunk
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[t][chunk]);
    };

    int g = 0;    // K/V blocks of the items so far: ring position
    int cs = 0;   // blocks of this tile so far: phase of its S / P hand-offs
    int no = 0;   // items in which this tile had blocks: phase of o_full
    bool ok = true;
    for (int n = 0; ok; ++n) {
      // the item stays in its ring slot until this warp is done with it: what the epilogue needs is derived
      // again after the block loop instead of being carried through it in registers
      int nbt, sk, shift, row, nb_max;
      {
        WorkItem it;
        ok = read_item(n, it, ctx);
        if (!(ok = __all_sync(0xffffffffu, ok))) break;
        if (it.mpair < 0) break;
        const Work w = decode_work(p, it);
        row = w.row0 + t * kBlockM + row_in_tile;
        nbt = t ? w.nb[1] : w.nb[0], sk = w.sk, shift = w.shift, nb_max = w.nb_max;
      }

      float m = -INFINITY;  // lazily updated reference maximum of the row (raw score units)
      float l = 0.f;        // row sum relative to m

      for (int j = 0; j < nbt; ++j) {
        // on behalf of the MMA thread (see there): the V block of this iteration and the K block of the next
        // have landed; both complete long before S(j), which this warp has to wait for in any case
        const int gj = g + j;
        if (!(ok = mbar_wait_warp(&bars->v_full[gj % C::kStages], (gj / C::kStages) & 1, ctx))) break;
        if (j + 1 < nbt &&
            !(ok = mbar_wait_warp(&bars->k_full[(gj + 1) % C::kStages], ((gj + 1) / C::kStages) & 1, ctx)))
          break;
        if (!(ok = mbar_wait_warp_hot(&bars->s_full[t], cs & 1, ctx))) break;
        ++cs;
        tc_fence_after_sync();

        // masking: only blocks that touch the sequence end or the causal diagonal
        const int col0 = j * kBlockN;
        int lim = sk - 1 - col0;  // last visible column index within this block
        if (p.is_causal) lim = min(lim, row + shift - col0);
        const bool masked = lim < kBlockN - 1;
        auto mask32 = [&](uint32_t (&v)[32], int base) {
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (base + i > lim) v[i] = 0xff800000u;
          }
        };
        // four independent chains: a single running maximum would be bound by the latency of 64 dependent ops
        auto max32 = [&](const uint32_t (&v)[32], float a) {
          float a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            a = fmax3(a, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            a1 = fmax3(a1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            a2 = fmax3(a2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            a3 = fmax3(a3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
          }
          return fmaxf(fmax3(a, a1, a2), a3);
        };

        // ---- pass 1: row maximum over all 128 columns, one round of loads ----
        uint32_t s0[32], s1[32];
        float mx = -INFINITY;
        {
          uint32_t s2[32], s3[32];
          tmem_ld32(tS + 64, s2);
          tmem_ld32(tS + 96, s3);
          tmem_ld32(tS, s0);
          tmem_ld32(tS + 32, s1);
          tmem_wait_ld();
          mask32(s2, 64);
          mask32(s3, 96);
          mx = max32(s3, max32(s2, mx));
          // the second read of these columns (pass 2) then needs no mask of its own; the stores are
          // warp-collective, so the decision is taken for the warp (`masked` differs between its rows)
          if (__any_sync(0xffffffffu, masked)) {
            tmem_st32(tS + 64, s2);
            tmem_st32(tS + 96, s3);
            tmem_wait_st();
          }
        }
        mask32(s0, 0);
        mask32(s1, 32);
        mx = max32(s1, max32(s0, mx));

        // lazy reference maximum, branch-free
        const bool fresh = (m == -INFINITY);
        const bool need = !fresh && (mx - m) * c > kRescaleThreshold;
        const float alpha = need ? ex2f((m - mx) * c) : 1.f;
        m = (fresh || need) ? mx : m;
        if (__any_sync(0xffffffffu, need)) {
          // S(j) complete implies that the PV MMAs of block j-1 have finished accumulating into O
          l *= alpha;
#pragma unroll 1
          for (int q = 0; q < D / 32; ++q) {
            uint32_t orr[32];
            tmem_ld32(tO + q * 32, orr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(tO + q * 32, orr);
          }
        }

        // ---- pass 2: P = exp2(S*c - m*c), row sum, fp16 P written over the consumed S columns ----
        const float nm = (m == -INFINITY) ? 0.f : -m * c;
        const float2 c2 = make_float2(c, c), nm2 = make_float2(nm, nm);
        float2 sum[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        // 32 keys -> 16 packed columns at column 16 * part of the S region
        auto exp_store = [&](const uint32_t (&v)[32], int part) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = ffma2(make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), c2, nm2);
            const float2 e = make_float2(ex2f(x.x), ex2f(x.y));
            sum[i & 3] = fadd2(sum[i & 3], e);  // independent chains, as for the maximum
            pk[i] = pack_half2(e.x, e.y);
          }
          tmem_st16(tS + part * 16, pk);
        };
        {
          uint32_t s2[32], s3[32];
          tmem_ld32(tS + 64, s2);  // in flight while the first 64 keys are exponentiated
          tmem_ld32(tS + 96, s3);
          exp_store(s0, 0);
          exp_store(s1, 1);
          hand_over(0);
          tmem_wait_ld();
          exp_store(s2, 2);
          exp_store(s3, 3);
          hand_over(1);
        }
        const float2 s01 = fadd2(sum[0], sum[1]), s23 = fadd2(sum[2], sum[3]);
        l += (s01.x + s01.y) + (s23.x + s23.y);
      }
      if (!ok) break;

      // ---- epilogue: O / l -> fp16, LSE; all thread-local.  The stores are not waited for: the next item's
      // softmax starts right behind them, and its first PV MMA (which overwrites O) is issued only after
      // this warp has handed over the next P, i.e. after these TMEM loads have completed. ----
      WorkItem it;
      {
        const volatile int* src = reinterpret_cast<const volatile int*>(&bars->items[n % kSchedDepth]);
        it.batch = src[0], it.head = src[1], it.mpair = src[2], it.pad = 0;
      }
      const Work w = decode_work(p, it);
      const bool row_valid = row < w.sq;
      int64_t o_index;
      if (varlen_q) {
        o_index = static_cast<int64_t>(w.q_off + row) * p.o_row_stride + w.head * p.o_head_stride;
      } else {
        o_index = w.batch * p.o_batch_stride + static_cast<int64_t>(row) * p.o_row_stride +
                  w.head * p.o_head_stride;
      }
      __half* orow = p.o + o_index;
      if (nbt > 0) {
        if (!(ok = mbar_wait_warp(&bars->o_full[t], no & 1, ctx))) break;
        ++no;
      }
      if (w.row0 + t * kBlockM < w.sq) {
        float lse_val = 0.f;
        float inv = 0.f;
        if (nbt > 0 && l > 0.f && m != -INFINITY) {
          inv = 1.f / l;
          lse_val = (m * c + __log2f(l)) * kLn2;
        }
        if (nbt > 0) {
          tc_fence_after_sync();
#pragma unroll 1
          for (int q = 0; q < D / 32; ++q) {
            uint32_t orr[32];
            tmem_ld32(tO + q * 32, orr);
            tmem_wait_ld();
            if (row_valid) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 v;
                v.x = pack_half2(__uint_as_float(orr[8 * i + 0]) * inv, __uint_as_float(orr[8 * i + 1]) * inv);
                v.y = pack_half2(__uint_as_float(orr[8 * i + 2]) * inv, __uint_as_float(orr[8 * i + 3]) * inv);
                v.z = pack_half2(__uint_as_float(orr[8 * i + 4]) * inv, __uint_as_float(orr[8 * i + 5]) * inv);
                v.w = pack_half2(__uint_as_float(orr[8 * i + 6]) * inv, __uint_as_float(orr[8 * i + 7]) * inv);
                *reinterpret_cast<uint4*>(orow + q * 32 + i * 8) = v;
              }
            }
          }
          tc_fence_before_sync();
        } else if (row_valid) {
          // no key block is visible to any row of this tile (causal with seqlen_q > seqlen_k)
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint4*>(orow + i * 8) = z;
        }
        if (row_valid) p.lse[(static_cast<int64_t>(w.batch) * p.h + w.head) * p.lse_row_stride + row] = lse_val;
      }
      g += nb_max;
      __syncwarp();
      if (lane == 0) release_item(n);
    }
  }

  // ---- common exit ----
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    // let TMA copies that may still be in flight land before the shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D>
int launch_fwd(FwdKernelParams& kp, int b, int h, int seqlen_q, int64_t total_q, cudaStream_t stream) {
  using C = Cfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FA_CHECK_CUDA(cudaFuncSetAttribute(fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       C::kSmemBytes));
    configured[dev & 63] = true;
  }
  const int sms = device_sm_count();
  kp.sched = next_sched_slot();
  if (sms <= 0 || kp.sched == nullptr) return set_error(FA_ERR_CUDA, "fa_fwd: device attributes not available");
  kp.items_x = (seqlen_q + kTiles * kBlockM - 1) / (kTiles * kBlockM);
  kp.b = b;
  const int64_t total = kp.cu_seqlens_q ? static_cast<int64_t>(h) * (total_q / (kTiles * kBlockM) + b)
                                        : static_cast<int64_t>(kp.items_x) * h * b;
  FA_CHECK_ARG(total < (1ll << 30), "fa_fwd: too many work items");
  kp.total_items = static_cast<int>(total);
  const int grid = kp.total_items < sms ? kp.total_items : sms;  // one CTA per SM (202 KB of shared memory each)
  fwd_kernel<D><<<grid, kNumThreads, C::kSmemBytes, stream>>>(kp);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

}  // namespace
}  // namespace fa

namespace fa {

int run_fwd(const FaFwdParams* p, int seqused_k_add, cudaStream_t stream) {
  FA_CHECK_ARG(p != nullptr, "fa_fwd: params is NULL");
  FA_CHECK_ARG(p->q && p->k && p->v && p->o && p->lse, "fa_fwd: q, k, v, o, lse must be non-NULL");
  if (p->d != 64 && p->d != 128)
    return set_error(FA_ERR_UNSUPPORTED, "fa_fwd: head_dim must be 64 or 128");
  FA_CHECK_ARG(p->b >= 1 && p->h >= 1 && p->h_k >= 1, "fa_fwd: b, h, h_k must be positive");
  FA_CHECK_ARG(p->h % p->h_k == 0, "fa_fwd: h must be divisible by h_k");
  FA_CHECK_ARG(p->seqlen_q >= 1 && p->seqlen_k >= 0, "fa_fwd: bad sequence lengths");
  FA_CHECK_ARG((p->cu_seqlens_q == nullptr) == (p->cu_seqlens_k == nullptr) || p->cu_seqlens_k == nullptr,
               "fa_fwd: cu_seqlens_k requires cu_seqlens_q");
  FA_CHECK_ARG(aligned16(p->o) && p->o_row_stride % 8 == 0 && p->o_head_stride % 8 == 0 &&
                   (p->cu_seqlens_q || p->o_batch_stride % 8 == 0),
               "fa_fwd: o must be 16-byte aligned with strides that are multiples of 8 elements");
  FA_CHECK_ARG(p->lse_row_stride >= p->seqlen_q, "fa_fwd: lse_row_stride is smaller than seqlen_q");
  FA_CHECK_ARG(p->is_causal >= 0 && p->is_causal <= 2, "fa_fwd: is_causal must be 0, 1 or FA_CAUSAL_SHIFT");
  FA_CHECK_ARG(p->is_causal != 2 || (!p->cu_seqlens_q && !p->seqused_k && !p->block_table),
               "fa_fwd: FA_CAUSAL_SHIFT is for dense q / k / v only");
  if (p->block_table) {
    FA_CHECK_ARG(p->page_size >= 128 && p->page_size % 128 == 0,
                 "fa_fwd: page_size must be a positive multiple of 128");
    FA_CHECK_ARG(!p->cu_seqlens_k && !p->cache_batch_idx,
                 "fa_fwd: block_table excludes cu_seqlens_k and cache_batch_idx");
    FA_CHECK_ARG(p->seqused_k != nullptr, "fa_fwd: block_table requires seqused_k");
  }
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;

  FwdKernelParams kp;
  const bool varlen_q = p->cu_seqlens_q != nullptr;
  const bool varlen_k = p->cu_seqlens_k != nullptr;
  const int64_t q_rows = varlen_q ? p->total_q : p->seqlen_q;
  const int64_t q_batch = varlen_q ? 1 : p->b;
  FA_CHECK_ARG(q_rows >= 1, "fa_fwd: q has no rows");
  rc = make_tensor_map_4d(&kp.tm_q, p->q, p->d, p->h, q_rows, q_batch, p->q_head_stride,
                          p->q_row_stride, p->q_batch_stride, kBlockM, "fa_fwd: q");
  if (rc != FA_OK) return rc;
  int64_t k_rows, k_batch;
  if (p->block_table) {
    k_rows = p->page_size;
    k_batch = p->k_batch;
  } else if (varlen_k) {
    k_rows = p->total_k;
    k_batch = 1;
  } else {
    k_rows = p->seqlen_k;
    k_batch = p->k_batch > 0 ? p->k_batch : p->b;
  }
  if (k_rows < 1) k_rows = 1;  // seqlen_k == 0: nothing is ever loaded
  rc = make_tensor_map_4d(&kp.tm_k, p->k, p->d, p->h_k, k_rows, k_batch, p->k_head_stride,
                          p->k_row_stride, p->k_batch_stride, kBlockN, "fa_fwd: k");
  if (rc != FA_OK) return rc;
  rc = make_tensor_map_4d(&kp.tm_v, p->v, p->d, p->h_k, k_rows, k_batch, p->v_head_stride,
                          p->v_row_stride, p->v_batch_stride, kBlockN, "fa_fwd: v");
  if (rc != FA_OK) return rc;

  kp.o = static_cast<__half*>(p->o);
  kp.lse = p->lse;
  kp.o_batch_stride = p->o_batch_stride;
  kp.o_row_stride = p->o_row_stride;
  kp.o_head_stride = p->o_head_stride;
  kp.lse_row_stride = p->lse_row_stride;
  kp.seqlen_q = p->seqlen_q;
  kp.seqlen_k = p->seqlen_k;
  kp.h = p->h;
  kp.h_k = p->h_k;
  kp.scale = p->softmax_scale;
  kp.scale_log2 = p->softmax_scale * kLog2e;
  kp.is_causal = p->is_causal;
  kp.causal_shift = p->causal_shift;
  kp.cu_seqlens_q = p->cu_seqlens_q;
  kp.cu_seqlens_k = p->cu_seqlens_k;
  kp.seqused_k = p->seqused_k;
  kp.seqused_k_add = seqused_k_add;
  kp.k_capacity = (p->block_table && p->block_table_cols > 0) ? p->block_table_cols * p->page_size
                  : (p->block_table ? 0x7fffffff : static_cast<int>(k_rows));
  kp.cache_batch_idx = p->cache_batch_idx;
  kp.block_table = p->block_table;
  kp.block_table_batch_stride = p->block_table_batch_stride;
  kp.page_size = p->page_size;
  kp.status = device_status_ptr();

  if (p->d == 128) return launch_fwd<128>(kp, p->b, p->h, p->seqlen_q, p->total_q, stream);
  return launch_fwd<64>(kp, p->b, p->h, p->seqlen_q, p->total_q, stream);
}

}  // namespace fa

extern "C" int fa_fwd(const FaFwdParams* p, fa_stream_t stream) {
  return fa::run_fwd(p, 0, static_cast<cudaStream_t>(stream));
}
