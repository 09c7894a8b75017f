// Backward attention for sm_100a as ONE kernel with the five algorithmic products (the two-kernel path of
// bwd_sm100.cu computes S and dP twice: seven products), plus a small pass that converts the fp32 dQ
// accumulator to fp16.
//
// One CTA owns a 128-key tile of one KV head and loops over the query heads of its GQA group and their
// Q tiles.  Per (key tile, Q tile) pair:
//     S^T  = K Q_i^T                  SS, fp32 in TMEM region S
//     dP^T = V dO_i^T                 SS, fp32 in TMEM region DP
//     P^T  = exp2(S^T c - lse2)       elementwise warps; fp16, written over the consumed S^T (TMEM)
//     dS^T = P^T o (dP^T - delta)     elementwise warps; fp16, written to SHARED memory, keys x queries
//     dV  += P^T dO_i                 TS (A = P^T from TMEM)
//     dK  += dS^T Q_i                 SS (A = the dS^T tile read K-major)
//     dQ_i partial = dS K             SS (A = the same dS^T tile read MN-major, B = K MN-major); fp32 into
//                                     the TMEM region of dP^T, which is free once dP^T sits in registers
// The dQ partial of a pair is read from TMEM by the elementwise warps themselves one pair later, right after they
// have handed over P^T of the next pair (one 16x256b load per warp: the 16 warps cover the 128 x D tile), and added
// to an fp32 accumulator in global memory with 16-byte reductions (red.global.add.v4.f32); the accumulator is laid
// out in the order of the TMEM fragments, so a warp's reduction writes 512 contiguous bytes, and the accumulator of
// a head stays resident in L2 while its key tiles are processed (measured: the 17 GB of reduction traffic of the
// benchmark shape never reach DRAM).  The TMEM region is handed back before the first reduction is issued.  The
// order of the additions depends on scheduling: dQ is NOT bitwise reproducible run to run (dK, dV are).
//
// This kernel is selected with FA_BWD_SINGLE_KERNEL; the default is the two-kernel path of bwd_sm100.cu, which is
// bitwise reproducible AND faster on B200 although it executes seven products instead of five: the 64 KB of
// reductions per pair leave the SM through its load/store unit at about one 32-byte sector per clock (~2000
// clocks per pair, the `lg_throttle` stall of the profile), and the warps that issue them are the ones the next
// pair waits for; without the reductions the kernel takes 6.4 ms at B4 S8192 H32 D128, with them 7.4 ms, the two
// kernels 2.9 + 4.2 ms.  A bulk reduction from shared memory would bypass that unit, but at head size 128 the
// tiles leave no shared memory to stage it.
//
// Warp roles (608 threads, 96 registers): warps 0-15 elementwise math, thread = (key row, 32-query column
// quarter); warp 16 TMA producer; warp 17 issues S^T and dP^T (the products the elementwise warps wait for) and
// owns the TMEM allocation; warp 18 issues dV, the dQ partial and dK.
// TMEM columns: S^T [0,128) with packed P^T over [0,64); dP^T / dQ partial [128,256); dV [256,256+D);
// dK [256+D, 256+2D).
//
// Replaces compute_dq_1rowblock and compute_dk_dv_1colblock (csrc/flash_attn/src/flash_bwd_kernel.h:25-609,
// 613-1344), their launches (src/flash_bwd_launch_template.h:84-138) and the GQA group sum
// (csrc/flash_attn/flash_api.cpp:338-348) of the reference.
#include "bwd_common.cuh"

namespace fa {
namespace {

constexpr int kFThreads = 608;  // 19 warps: five on one SM sub-partition -> 96 registers per thread
constexpr int kFComputeWarps = 16;
constexpr int kFProducerWarp = 16;
constexpr int kFMmaWarpA = 17;
constexpr int kFMmaWarpB = 18;
constexpr int kFColS = 0;
constexpr int kFColDP = 128;
constexpr int kFColAcc = 256;
static_assert((kFThreads / 32 + 3) / 4 * 32 * 96 <= 16384, "register file of one SM sub-partition");

template <int D>
struct FCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kDsBytes = 2 * kChunkBytes;        // 128 keys x 128 queries fp16
  static constexpr int kStagesQ = (D == 128) ? 2 : 3;
  static constexpr int kStagesDO = (D == 128) ? 2 : 3;
  static constexpr int kAlignPad = (D == 128) ? 0 : 1024;  // head size 128: 224 KB of tiles, no room for a pad
  static constexpr int kSmemBytes = 2 * kTileBytes + kDsBytes + (kStagesQ + kStagesDO) * kTileBytes + 2048 /*stats*/ +
                                    512 /*barriers*/ + kAlignPad;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct FBarriers {
  uint64_t kv_full;
  uint64_t q_full[4], q_empty[4];    // q_empty: two readers (S^T issuer, dK issuer)
  uint64_t do_full[4], do_empty[4];  // do_empty: two readers (dP^T issuer, dV issuer)
  uint64_t st_full[2], st_empty[2];  // row statistics of a Q tile
  uint64_t s_full, dp_full;          // accumulators ready for the elementwise warps
  uint64_t p_full, ds_full;          // packed P^T in TMEM / dS^T in shared memory written by all 16 warps
  uint64_t s_read[4];                // per TMEM lane quarter: its four column-quarter warps hold their S^T values
  uint64_t p_used;                   // dV MMAs have consumed P^T: region S may receive the next S^T
  uint64_t ds_used;                  // dQ and dK MMAs have consumed the dS^T tile
  uint64_t dq_full;                  // dQ partial complete in TMEM
  uint64_t dq_read;                  // ... and read by the 16 elementwise warps: region DP may receive dP^T
  uint64_t tail_fixed[4];            // per dO stage: rows past the end of a packed sequence zeroed in Q and dO
  uint64_t k_fixed;                  // rows past the end of a packed sequence zeroed in the K tile
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(FBarriers) <= 512, "barrier block");

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <int D, bool kVarlen>
__global__ void __launch_bounds__(kFThreads, 1)
bwd_fused_kernel(const __grid_constant__ BwdKernelParams p) {
  using C = FCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int batch = blockIdx.z, head_k = blockIdx.y, nblk = blockIdx.x;
  constexpr bool varlen = kVarlen;
  const int q_off = varlen ? p.cu_seqlens_q[batch] : 0;
  const int sq = varlen ? p.cu_seqlens_q[batch + 1] - q_off : p.seqlen_q;
  const int k_off = varlen ? p.cu_seqlens_k[batch] : 0;
  const int sk = varlen ? p.cu_seqlens_k[batch + 1] - k_off : p.seqlen_k;
  const int key0 = nblk * kBlock;
  if (key0 >= sk) return;
  if (cta_should_stop(p.status)) return;
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
  uint8_t* sDS = sV + C::kTileBytes;
  uint8_t* sQ = sDS + C::kDsBytes;
  uint8_t* sdO = sQ + C::kStagesQ * C::kTileBytes;
  float* sStats = reinterpret_cast<float*>(sdO + C::kStagesDO * C::kTileBytes);  // [2][lse2 128 | delta 128]
  FBarriers* bars = reinterpret_cast<FBarriers*>(reinterpret_cast<uint8_t*>(sStats) + 2048);
  if (smem - smem_raw > C::kAlignPad) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusSmemLayout);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // tag: 1 elementwise warp, 2 producer, 3 issuer of S^T / dP^T, 4 issuer of dV / dQ / dK
  WaitCtx ctx{&bars->abort_flag, p.status, warp < kFComputeWarps ? 1 : warp - kFProducerWarp + 2, bars};
  auto load_q_do = [&](int it) -> bool {
    const int sq_ = it % C::kStagesQ, sd = it % C::kStagesDO, ss = it & 1;
    const uint32_t phq = (it / C::kStagesQ) & 1, phd = (it / C::kStagesDO) & 1, phs = (it >> 1) & 1;
    const int head = head_k * group + it / per_head;
    const int i = i_min + it % per_head;
    const int qrow = q_off + i * kBlock;
    const int64_t stat = (static_cast<int64_t>(batch) * p.h + head) * p.sq_pad + i * kBlock;
    if (!mbar_wait(&bars->q_empty[sq_], phq ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->q_full[sq_], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sQ + sq_ * C::kTileBytes + c * C::kChunkBytes, &p.tm_q, &bars->q_full[sq_], c * 64, head, qrow, bq);
    if (!mbar_wait(&bars->st_empty[ss], phs ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->st_full[ss], 1024);
    bulk_load_1d(sStats + ss * 256, p.lse2 + stat, 512, &bars->st_full[ss]);
    bulk_load_1d(sStats + ss * 256 + 128, p.delta + stat, 512, &bars->st_full[ss]);
    if (!mbar_wait(&bars->do_empty[sd], phd ^ 1, ctx)) return false;
    mbar_arrive_expect_tx(&bars->do_full[sd], C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kChunks; ++c)
      tma_load_4d(sdO + sd * C::kTileBytes + c * C::kChunkBytes, &p.tm_do, &bars->do_full[sd], c * 64, head, qrow, bq);
    return true;
  };
  const int n_early = min(n_it, 2);  // stages that are free from the start: no wait blocks
  if (warp == kFProducerWarp && lane == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 2);
      mbar_init(&bars->do_full[s], 1);
      mbar_init(&bars->do_empty[s], 2);
      mbar_init(&bars->tail_fixed[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->st_full[s], 1);
      mbar_init(&bars->st_empty[s], kFComputeWarps);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, kFComputeWarps);
    mbar_init(&bars->ds_full, kFComputeWarps);
    for (int s = 0; s < 4; ++s) mbar_init(&bars->s_read[s], 4);
    mbar_init(&bars->p_used, 1);
    mbar_init(&bars->ds_used, 1);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_read, kFComputeWarps);
    mbar_init(&bars->k_fixed, 1);
    mbar_init(&bars->acc_full, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    if (n_it > 0) {
      mbar_arrive_expect_tx(&bars->kv_full, 2 * C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(sK + c * C::kChunkBytes, &p.tm_k, &bars->kv_full, c * 64, head_k, k_off + key0, bq);
        tma_load_4d(sV + c * C::kChunkBytes, &p.tm_v, &bars->kv_full, c * 64, head_k, k_off + key0, bq);
      }
      for (int it = 0; it < n_early; ++it) load_q_do(it);
    }
  }
  if (warp == kFMmaWarpA) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  // packed sequences: the last Q / dO tile and the K tile may hold rows of the next sequence
  const bool fix_q_tail = kVarlen && (sq % kBlock) != 0 && n_it > 0;
  const int q_tail_rows = sq - (nq - 1) * kBlock;  // valid rows of the last Q tile
  const bool fix_k_tail = kVarlen && key0 + kBlock > sk && n_it > 0;

  if (warp < kFComputeWarps) {
    // ---- elementwise warps: thread = (key row, 32-query-column quarter) ----
    const int cq = warp >> 2, quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int key = key0 + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kFColS + cq * 32;     // S^T
    const uint32_t tDP = tmem_base + lane_base + kFColDP + cq * 32;   // dP^T
    const uint32_t tP = tmem_base + lane_base + kFColS + cq * 16;     // packed P^T
    // dS^T tile in shared memory: row = key (128 bytes = 64 queries), two 64-query chunks, 128-byte swizzle
    // (16-byte unit u of row r sits at unit u ^ (r % 8)): the layout TMA writes, so the tile can be read as a
    // K-major A operand (dK) and as an MN-major A operand (dQ)
    const uint32_t ds_row = smem_u32(sDS) + (cq >> 1) * C::kChunkBytes + row_in_tile * 128;
    const int ds_unit0 = (cq & 1) * 4;
    const int sw = row_in_tile & 7;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    const int cmin0 = p.is_causal ? key - shift - (i_min * kBlock + cq * 32) : 0;
    const float* stats = sStats + cq * 32;
    const int cmax_last = fix_q_tail ? max(0, min(32, q_tail_rows - cq * 32)) : 32;  // valid columns in the last Q tile
    int i_rel = 0;  // Q tile within the current head
    const int64_t acc_tile0 = dq_acc_tile_base(p, batch, q_off);
    // ---- dQ partial of pair `it`: TMEM -> fp32 accumulator in global memory ----
    // Warp (quarter, cq) takes TMEM lanes 16 * (cq & 1) .. +15 of its quarter and columns (cq >> 1) * (D / 2) ..
    // + D / 2 - 1 with one 16x256b load: thread (g = lane / 4, t = lane % 4) gets, per repetition j, columns 8j + 2t,
    // 8j + 2t + 1 of lanes g and g + 8 -- four floats, added with ONE 16-byte reduction.  The accumulator tile is
    // stored in exactly this fragment order, so the 32 threads of a reduction write 512 contiguous bytes.  The TMEM
    // region is handed back (dq_read) before the first reduction is issued.
    auto drain_dq = [&](int it) -> bool {
      const int head = head_k * group + it / per_head;
      const int i = i_min + it % per_head;
      float* a = p.dq_acc + (static_cast<int64_t>(head) * p.dq_acc_rows + (acc_tile0 + i) * kBlock) * D +
                 ((quarter * 2 + (cq & 1)) * 2 + (cq >> 1)) * (16 * D / 2) + lane * 4;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32 + (cq & 1) * 16) << 16) + kFColDP + (cq >> 1) * (D / 2);
      if (!mbar_wait_warp(&bars->dq_full, it & 1, ctx)) return false;
      tc_fence_after_sync();
      uint32_t r[D / 4];
      if constexpr (D == 128) tmem_ld_16x256b_x8(taddr, r); else tmem_ld_16x256b_x4(taddr, r);
      tmem_wait_ld();
      warp_arrive_loaded(&bars->dq_read, lane);  // region DP may receive the next dP^T
#pragma unroll
      for (int j = 0; j < D / 16; ++j)
        red_add_v4(a + 128 * j, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                   __uint_as_float(r[4 * j + 3]));
      return true;
    };
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int ss = it & 1;
      ctx.iter = it;
      if (!(ok = mbar_wait_warp(&bars->st_full[ss], (it >> 1) & 1, ctx))) break;
      const float4* st_lse = reinterpret_cast<const float4*>(stats + ss * 256);
      const float4* st_delta = reinterpret_cast<const float4*>(stats + ss * 256 + 128);
      constexpr bool kEarlyLse = (D == 128);  // fetched while the warp waits for S^T anyway (see bwd_sm100.cu)
      float4 lse_q[8];
      if constexpr (kEarlyLse) {
#pragma unroll
        for (int e = 0; e < 8; ++e) lse_q[e] = st_lse[e];
      }
      if (!(ok = mbar_wait_warp(&bars->s_full, it & 1, ctx))) break;
      tc_fence_after_sync();
      uint32_t sr[32];
      tmem_ld32(tS, sr);
      tmem_wait_ld();
      // P^T is written over S^T: the four column-quarter warps of this lane quarter announce that they hold
      // their S^T values; the rendezvous completes under the exponentials and is checked before the store
      warp_arrive_loaded(&bars->s_read[quarter], lane);
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
      // rows of the key tile past the end of the sequence (key >= sk) hold no key: P = dS = 0 by selection
      const bool key_dead = key >= sk;
      if (col_masked || key_dead) {
        const int cmin = key_dead ? 32 : (cmask & 0xff), cmax = cmask >> 8;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (2 * e < cmin || 2 * e >= cmax) pr[e].x = 0.f;
          if (2 * e + 1 < cmin || 2 * e + 1 >= cmax) pr[e].y = 0.f;
        }
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) pk[e] = pack_half2(pr[e].x, pr[e].y);
      if (!(ok = warp_wait_unless(warp_probe(&bars->s_read[quarter], it & 1), &bars->s_read[quarter], it & 1, ctx))) break;
      tc_fence_after_sync();
      tmem_st16(tP, pk);
      warp_arrive(&bars->p_full, lane);
      // The dQ partial of the PREVIOUS pair is drained here: its product finished long ago (no waiting), and the
      // reductions are issued while dP^T of this pair, which needs the region the partial occupied, is computed.
      // (Draining at the end of the pair's own iteration makes the warps wait ~1400 clocks for the dQ product
      // and was 5 % slower.)
      if (it > 0 && !(ok = drain_dq(it - 1))) break;

      if (!(ok = mbar_wait_warp(&bars->dp_full, it & 1, ctx))) break;
      tc_fence_after_sync();
      tmem_ld32(tDP, sr);
      tmem_wait_ld();
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
      if (col_masked || key_dead) {  // by selection: dP^T of a masked position may be NaN/Inf (rows of another sequence)
        const int cmin = key_dead ? 32 : (cmask & 0xff), cmax = cmask >> 8;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (2 * e < cmin || 2 * e >= cmax) pk[e] &= 0xffff0000u;
          if (2 * e + 1 < cmin || 2 * e + 1 >= cmax) pk[e] &= 0x0000ffffu;
        }
      }
      // the statistics of this tile are in use no longer
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->st_empty[ss]);
      // the dQ and dK MMAs of the previous pair must have consumed the old dS^T tile
      if (it > 0 && !(ok = mbar_wait_warp(&bars->ds_used, (it - 1) & 1, ctx))) break;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        st_shared_v4(ds_row + (((ds_unit0 + u) ^ sw) << 4), pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
      // the arrival also tells the MMA warp that this warp has read dP^T: region DP may receive the dQ partial
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_full);
    }
    if (ok && n_it > 0) ok = drain_dq(n_it - 1);
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
          tmem_ld32(tmem_base + lane_base + kFColAcc + which * D + col_half * (D / 2) + q * 32, r);
          tmem_wait_ld();
          if (key < sk) store_row_fp16(dst + q * 32, r, mul);
        }
      } else if (key < sk) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i3 = 0; i3 < D / 16; ++i3) *reinterpret_cast<uint4*>(dst + i3 * 8) = z;
      }
    }
  } else {
    if (warp == kFProducerWarp) {
      // =========================== TMA producer ===========================
      if (fix_k_tail) {
        if (mbar_wait_warp(&bars->kv_full, 0, ctx)) {
          // (zero_tile_rows_from is written for BCfg<D>: same chunk geometry)
          zero_tile_rows_from<D>(sK, sk - key0, lane);
          if (lane == 0) mbar_arrive(&bars->k_fixed);
        }
      }
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
            if (!mbar_wait_warp(&bars->q_full[sq_], (it / C::kStagesQ) & 1, ctx)) break;
            if (!mbar_wait_warp(&bars->do_full[sd], (it / C::kStagesDO) & 1, ctx)) break;
            zero_tile_rows_from<D>(sQ + sq_ * C::kTileBytes, q_tail_rows, lane);
            zero_tile_rows_from<D>(sdO + sd * C::kTileBytes, q_tail_rows, lane);
            if (lane == 0) mbar_arrive(&bars->tail_fixed[sd]);
          }
        }
      }
    } else if (warp == kFMmaWarpA) {
      if (lane == 0 && n_it > 0) {
        constexpr uint32_t idesc_nn = make_idesc_f16(128, kBlock, false, false);
        const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
        auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, ctx); };
        auto q_tile = [&](int it) { return smem_u32(sQ + (it % C::kStagesQ) * C::kTileBytes); };
        auto do_tile = [&](int it) { return smem_u32(sdO + (it % C::kStagesDO) * C::kTileBytes); };
        auto q_full = [&](int it) { return wait(&bars->q_full[it % C::kStagesQ], (it / C::kStagesQ) & 1); };
        auto do_full = [&](int it) { return wait(&bars->do_full[it % C::kStagesDO], (it / C::kStagesDO) & 1); };
        bool ok = wait(&bars->kv_full, 0) && q_full(0);
        for (int it = 0; ok && it < n_it; ++it) {
          ctx.iter = it;
          // region S holds P^T of the previous pair until its dV MMAs are done
          if (it > 0 && !(ok = wait(&bars->p_used, (it - 1) & 1))) break;
          tc_fence_after_sync();
          ok = gemm_ss<D>(tmem_base + kFColS, k_addr, q_tile(it), idesc_nn, [&] { return do_full(it); });  // S^T = K Q^T
          if (!ok) break;
          tc_commit(&bars->s_full);
          tc_commit(&bars->q_empty[it % C::kStagesQ]);  // second reader: the dK MMAs of this pair
          // region DP holds the dQ partial of the previous pair until the reduction warps have read it
          if (it > 0 && !(ok = wait(&bars->dq_read, (it - 1) & 1))) break;
          tc_fence_after_sync();
          ok = gemm_ss<D>(tmem_base + kFColDP, v_addr, do_tile(it), idesc_nn,  // dP^T = V dO^T
                          [&] { return it + 1 >= n_it || q_full(it + 1); });
          if (!ok) break;
          tc_commit(&bars->dp_full);
          tc_commit(&bars->do_empty[it % C::kStagesDO]);  // second reader: the dV MMAs of this pair
        }
      }
    } else if (warp == kFMmaWarpB) {
      if (lane == 0 && n_it > 0) {
        constexpr uint32_t idesc_dv = make_idesc_f16(128, D, false, true);   // A = P^T (TMEM), B = dO MN-major
        constexpr uint32_t idesc_dk = make_idesc_f16(128, D, false, true);   // A = dS^T K-major, B = Q MN-major
        constexpr uint32_t idesc_dq = make_idesc_f16(128, D, true, true);    // A = dS^T MN-major, B = K MN-major
        const uint32_t tP = tmem_base + kFColS, tDQ = tmem_base + kFColDP;
        const uint32_t tDV = tmem_base + kFColAcc, tDK = tmem_base + kFColAcc + D;
        // dS^T tile: 128 key rows of 128 bytes per 64-query chunk, chunks 16 KB apart
        const uint64_t ds_kmajor = make_smem_desc(smem_u32(sDS), 16, 1024);
        const uint64_t ds_mnmajor = make_smem_desc(smem_u32(sDS), C::kChunkBytes, 1024);
        const uint64_t k_mnmajor = mnmajor_tile<D>(smem_u32(sK));
        bool ok = true;
        uint32_t tail_phase = 0;  // bit sd: parity of the next tail_fixed[sd] phase to wait for
        for (int it = 0; ok && it < n_it; ++it) {
          ctx.iter = it;
          const int sq_ = it % C::kStagesQ, sd = it % C::kStagesDO;
          if (!(ok = mbar_wait(&bars->do_full[sd], (it / C::kStagesDO) & 1, ctx))) break;
          if (!(ok = mbar_wait(&bars->p_full, it & 1, ctx))) break;
          if (fix_q_tail && it % per_head == per_head - 1) {
            if (!(ok = mbar_wait(&bars->tail_fixed[sd], (tail_phase >> sd) & 1, ctx))) break;
            tail_phase ^= 1u << sd;
          }
          tc_fence_after_sync();
          gemm_ts<D>(tDV, tP, smem_u32(sdO + sd * C::kTileBytes), idesc_dv, it == 0);  // dV += P^T dO
          tc_commit(&bars->do_empty[sd]);
          tc_commit(&bars->p_used);
          if (!(ok = mbar_wait(&bars->q_full[sq_], (it / C::kStagesQ) & 1, ctx))) break;
          if (!(ok = mbar_wait(&bars->ds_full, it & 1, ctx))) break;
          if (fix_k_tail && it == 0 && !(ok = mbar_wait(&bars->k_fixed, 0, ctx))) break;
          tc_fence_after_sync();
          // dQ partial = dS K: contraction over the 128 keys in 8 slices of 16 rows (2048 B) of both tiles
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tDQ, desc_advance(ds_mnmajor, k * 2048), mnmajor_slice(k_mnmajor, k), idesc_dq, k > 0);
          tc_commit(&bars->dq_full);
          // dK += dS^T Q: contraction over the 128 queries; slice k of A = 32 bytes inside the 128-byte rows of
          // chunk k / 4, slice k of B = 16 rows of the Q tile
          const uint64_t q_mnmajor = mnmajor_tile<D>(smem_u32(sQ + sq_ * C::kTileBytes));
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tDK, desc_advance(ds_kmajor, (k >> 2) * C::kChunkBytes + (k & 3) * 32), mnmajor_slice(q_mnmajor, k),
                   idesc_dk, (it > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->q_empty[sq_]);
          tc_commit(&bars->ds_used);
        }
        if (ok) tc_commit(&bars->acc_full);
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
  if (warp == kFMmaWarpA) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dq = scale * accumulator, fp32 -> fp16.  The accumulator holds every 128-row tile in the fragment order of the
// read-out above: the tile is 16 blocks of 16 rows x D/2 columns (block = ((row / 32) * 2 + (row % 32) / 16) * 2 +
// col / (D / 2)), and inside a block the float at (row g or g + 8, column 8j + 2t + e) sits at
// j * 128 + (g * 4 + t) * 4 + (row >= 8 ? 2 : 0) + e.  One thread converts one 16-byte group (two columns of two
// rows); a warp reads 512 contiguous bytes.  grid (ceil(seqlen_q / 128), h, b), 256 threads, each 128 x D tile in
// D / 8 passes.
__global__ void __launch_bounds__(256)
bwd_dq_finalize_kernel(const float* __restrict__ acc, __half* __restrict__ dq, int64_t acc_rows, int sq_pad, int seqlen_q,
                       int d, const int* __restrict__ cu_seqlens_q, int64_t dq_batch_stride,
                       int64_t dq_row_stride, int64_t dq_head_stride, float scale) {
  const int batch = blockIdx.z, head = blockIdx.y, tile = blockIdx.x;
  const int q_off = cu_seqlens_q ? cu_seqlens_q[batch] : 0;
  const int sq = cu_seqlens_q ? cu_seqlens_q[batch + 1] - q_off : seqlen_q;
  if (tile * 128 >= sq) return;
  const int64_t tile0 = cu_seqlens_q ? static_cast<int64_t>(q_off / 128 + batch) : static_cast<int64_t>(batch) * (sq_pad / 128);
  const float4* src = reinterpret_cast<const float4*>(acc + (static_cast<int64_t>(head) * acc_rows + (tile0 + tile) * 128) * d);
  __half* dst = dq + (cu_seqlens_q ? static_cast<int64_t>(q_off) * dq_row_stride : batch * dq_batch_stride) + head * dq_head_stride;
  const int groups = 128 * d / 4;          // 16-byte groups per tile
  const int groups_per_block = 16 * (d / 2) / 4;
  for (int idx = threadIdx.x; idx < groups; idx += 256) {
    const float4 v = src[idx];
    const int blk = idx / groups_per_block, in_blk = idx % groups_per_block;
    const int j = in_blk / 32, lane = in_blk % 32, g = lane >> 2, t = lane & 3;
    const int row = tile * 128 + (blk >> 2) * 32 + ((blk >> 1) & 1) * 16 + g;
    const int col = (blk & 1) * (d / 2) + 8 * j + 2 * t;
    if (row < sq)
      *reinterpret_cast<uint32_t*>(dst + static_cast<int64_t>(row) * dq_row_stride + col) = pack_half2(v.x * scale, v.y * scale);
    if (row + 8 < sq)
      *reinterpret_cast<uint32_t*>(dst + static_cast<int64_t>(row + 8) * dq_row_stride + col) = pack_half2(v.z * scale, v.w * scale);
  }
}

template <int D>
int launch_fused(const BwdKernelParams& kp, const FaBwdParams* p, cudaStream_t stream) {
  using C = FCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  FA_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_fused_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    FA_CHECK_CUDA(cudaFuncSetAttribute(bwd_fused_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured[dev & 63] = true;
  }
  dim3 grid((p->seqlen_k + kBlock - 1) / kBlock, p->h_k, p->b);
  if (kp.cu_seqlens_q != nullptr)
    bwd_fused_kernel<D, true><<<grid, kFThreads, C::kSmemBytes, stream>>>(kp);
  else
    bwd_fused_kernel<D, false><<<grid, kFThreads, C::kSmemBytes, stream>>>(kp);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

}  // namespace

int launch_bwd_fused(const BwdKernelParams& kp, const FaBwdParams* p, cudaStream_t stream) {
  if (p->d == 128) return launch_fused<128>(kp, p, stream);
  return launch_fused<64>(kp, p, stream);
}

int launch_bwd_dq_finalize(const BwdKernelParams& kp, const FaBwdParams* p, cudaStream_t stream) {
  dim3 grid((p->seqlen_q + 127) / 128, p->h, p->b);
  bwd_dq_finalize_kernel<<<grid, 256, 0, stream>>>(kp.dq_acc, kp.dq, kp.dq_acc_rows, kp.sq_pad, p->seqlen_q, p->d,
                                                   kp.cu_seqlens_q, kp.dq_batch_stride, kp.dq_row_stride,
                                                   kp.dq_head_stride, kp.scale);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa
