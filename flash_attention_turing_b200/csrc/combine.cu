// Split-KV merge: LSE = logsumexp_s lse_s, O = sum_s exp(lse_s - LSE) * O_s.
//
// One warp per output row.  The split LSEs are spread over the lanes and reduced with warp
// shuffles (max, then sum of exponentials); each lane then owns D/32 consecutive output columns
// and streams the fp32 partial rows with 8- or 16-byte loads, so a row of every split is one
// fully coalesced 256/512-byte read.  HBM-bound: bytes = splits*rows*(D+1)*4 + rows*(2*D+4).
//
// Replaces kvcache_combine_kernel / kvcache_combine_kernel_legacy of the reference
// (csrc/flash_attn/src/kvcache_native.cu:676-780); rows whose every split is empty get O = 0 and
// LSE = 0 as there (:727).
#include "combine.h"

#define FA_WAIT_INLINE
#include "ptx.cuh"

namespace fa {
namespace {

constexpr int kWarpsPerBlock = 8;

template <int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
combine_kernel(const float* __restrict__ o_accum, const float* __restrict__ lse_accum,
               __half* __restrict__ o, float* __restrict__ lse, int64_t rows, int num_splits,
               int h, int seqlen_q, int64_t o_batch_stride, int64_t o_row_stride,
               int64_t o_head_stride) {
  constexpr int kPerLane = D / 32;  // 2 or 4 consecutive columns
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;

  // log-sum-exp over splits: lanes stride over the splits, shuffles reduce
  float mx = -INFINITY;
  for (int s = lane; s < num_splits; s += 32) mx = fmaxf(mx, lse_accum[s * rows + row]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float sum = 0.f;
  if (mx != -INFINITY)
    for (int s = lane; s < num_splits; s += 32) sum += __expf(lse_accum[s * rows + row] - mx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const bool empty = (mx == -INFINITY) || (sum == 0.f);
  const float lse_total = empty ? -INFINITY : mx + __logf(sum);

  float acc[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) acc[i] = 0.f;
  if (!empty) {
    for (int s = 0; s < num_splits; ++s) {
      const float ls = lse_accum[s * rows + row];  // same address for all lanes: one broadcast load
      if (ls == -INFINITY) continue;
      const float w = __expf(ls - lse_total);
      const float* src = o_accum + (static_cast<int64_t>(s) * rows + row) * D + lane * kPerLane;
      if constexpr (kPerLane == 4) {
        const float4 x = *reinterpret_cast<const float4*>(src);
        acc[0] = fmaf(w, x.x, acc[0]);
        acc[1] = fmaf(w, x.y, acc[1]);
        acc[2] = fmaf(w, x.z, acc[2]);
        acc[3] = fmaf(w, x.w, acc[3]);
      } else {
        const float2 x = *reinterpret_cast<const float2*>(src);
        acc[0] = fmaf(w, x.x, acc[0]);
        acc[1] = fmaf(w, x.y, acc[1]);
      }
    }
  }

  // rows are ordered (b, h, seqlen_q)
  const int64_t bh = row / seqlen_q;
  const int q_pos = static_cast<int>(row - bh * seqlen_q);
  const int64_t batch = bh / h;
  const int head = static_cast<int>(bh - batch * h);
  __half* dst = o + batch * o_batch_stride + q_pos * o_row_stride + head * o_head_stride +
                lane * kPerLane;
  if constexpr (kPerLane == 4) {
    uint2 v;
    v.x = pack_half2(acc[0], acc[1]);
    v.y = pack_half2(acc[2], acc[3]);
    *reinterpret_cast<uint2*>(dst) = v;
  } else {
    *reinterpret_cast<uint32_t*>(dst) = pack_half2(acc[0], acc[1]);
  }
  if (lse != nullptr && lane == 0) lse[row] = empty ? 0.f : lse_total;
}

// Merge over ranks with the partials read in place (possibly from peer GPUs): D/8 lanes per output row
// (b, row, h); the per-part LSEs sit in the lanes of the row's group and are reduced with shuffles, every lane then
// owns 8 consecutive columns of the fp16 partial rows (16-byte reads, a row is one contiguous 128 or 256 bytes).
__device__ __forceinline__ uint4 load16_if(const void* ptr, bool pred) {
  uint4 v = make_uint4(0, 0, 0, 0);
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "@p ld.global.v4.u32 {%0, %1, %2, %3}, [%4];\n\t"
      "}\n"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "l"(ptr), "r"(static_cast<int>(pred))
      : "memory");
  return v;
}

struct GatherArgs {
  const __half* o_part[FA_MAX_GATHER_PARTS];
  const float* lse_part[FA_MAX_GATHER_PARTS];
};

template <int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
combine_gather_kernel(const __grid_constant__ GatherArgs a, __half* __restrict__ o, float* __restrict__ lse,
                      int num_parts, int b, int h, int seqlen_q, int row_begin, int rows) {
  // D/8 lanes per output row, 16 bytes per lane: a warp merges 2 (D = 128) or 4 (D = 64) rows.  The parts of a
  // row are fetched in batches of eight loads issued back to back before any of them is used: the reads go to
  // other GPUs' memory over NVLink (microseconds of latency), so what matters is the number of bytes in flight.
  constexpr int kLanes = D / 8;           // lanes per row
  constexpr int kRows = 32 / kLanes;      // rows per warp
  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes, rsel = lane / kLanes;
  const int64_t total = static_cast<int64_t>(b) * rows * h;
  const int64_t idx = (static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5)) * kRows + rsel;
  const bool live = idx < total;
  const int64_t id = live ? idx : total - 1;  // dead lanes repeat the last row (shuffles need every lane)
  const int head = static_cast<int>(id % h);
  const int r = static_cast<int>((id / h) % rows);
  const int batch = static_cast<int>(id / (static_cast<int64_t>(h) * rows));
  const int64_t lse_idx = (static_cast<int64_t>(batch) * h + head) * seqlen_q + row_begin + r;
  const int64_t o_idx = ((static_cast<int64_t>(batch) * seqlen_q + row_begin + r) * h + head) * D + sub * 8;

  // the LSEs of the parts sit in the lanes of the row's group (part p in lane p and, for D = 64 with more than
  // eight parts, in a second round)
  float mx = -INFINITY;
  float my[(FA_MAX_GATHER_PARTS + kLanes - 1) / kLanes];
#pragma unroll
  for (int k = 0; k < (FA_MAX_GATHER_PARTS + kLanes - 1) / kLanes; ++k) {
    const int part = k * kLanes + sub;
    my[k] = (part < num_parts) ? a.lse_part[part][lse_idx] : -INFINITY;
    mx = fmaxf(mx, my[k]);
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float e[(FA_MAX_GATHER_PARTS + kLanes - 1) / kLanes];
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < (FA_MAX_GATHER_PARTS + kLanes - 1) / kLanes; ++k) {
    e[k] = (mx == -INFINITY || my[k] == -INFINITY) ? 0.f : __expf(my[k] - mx);
    sum += e[k];
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const bool empty = (mx == -INFINITY) || (sum == 0.f);
  const float inv = empty ? 0.f : 1.f / sum;

  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int p0 = 0; p0 < num_parts; p0 += 8) {
    uint4 raw[8];
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int part = p0 + i;  // uniform over the warp
      // weight of `part` for this lane's row: held by lane (part % kLanes) of the row's group in round part / kLanes
      float wk = 0.f;
#pragma unroll
      for (int k = 0; k < (FA_MAX_GATHER_PARTS + kLanes - 1) / kLanes; ++k) {
        const float v = __shfl_sync(0xffffffffu, e[k], rsel * kLanes + (part % kLanes));
        if (k == part / kLanes) wk = v;
      }
      w[i] = (part < num_parts) ? wk * inv : 0.f;
      // predicated, not branched: the eight loads of a batch are issued back to back; parts without keys for
      // this row (weight 0) are not read at all
      raw[i] = load16_if(part < num_parts ? a.o_part[part] + o_idx : nullptr, w[i] != 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&u[c]));
        acc[2 * c] = fmaf(w[i], x.x, acc[2 * c]);
        acc[2 * c + 1] = fmaf(w[i], x.y, acc[2 * c + 1]);
      }
    }
  }
  if (!live) return;
  uint4 v;
  v.x = pack_half2(acc[0], acc[1]);
  v.y = pack_half2(acc[2], acc[3]);
  v.z = pack_half2(acc[4], acc[5]);
  v.w = pack_half2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(o + ((static_cast<int64_t>(batch) * rows + r) * h + head) * D + sub * 8) = v;
  if (sub == 0) lse[(static_cast<int64_t>(batch) * h + head) * rows + r] = empty ? 0.f : mx + __logf(sum);
}

// out[b, r, :] = sum over parts of part[b, row_begin + r, :] (fp32 sum of fp16 values); one thread per 8
// consecutive values of a row of h * d.
struct SumArgs {
  const __half* part[FA_MAX_GATHER_PARTS];
  int first_row[FA_MAX_GATHER_PARTS];  // rows below hold nothing in this part: not read
};
__global__ void __launch_bounds__(256)
sum_gather_kernel(const __grid_constant__ SumArgs a, __half* __restrict__ out, int num_parts, int64_t total_vec,
                  int64_t vec_per_slice, int64_t vec_per_seq, int64_t vec_row_begin, int64_t vec_per_row, int row_begin) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int64_t batch = idx / vec_per_slice;
  const int64_t in_slice = idx - batch * vec_per_slice;
  const int64_t src = batch * vec_per_seq + vec_row_begin + in_slice;
  const int row = row_begin + static_cast<int>(in_slice / vec_per_row);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // eight predicated loads issued back to back per batch (the parts may be other GPUs' memory: what matters is
  // the number of bytes in flight); a part is not read below its first valid row.  The additions keep the order
  // of the parts, so the result does not depend on the batching.
  for (int p0 = 0; p0 < num_parts; p0 += 8) {
    uint4 raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int part = p0 + i;
      const bool use = part < num_parts && row >= a.first_row[part & (FA_MAX_GATHER_PARTS - 1)];
      raw[i] = load16_if(use ? reinterpret_cast<const uint4*>(a.part[part]) + src : nullptr, use);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&w[c]));
        acc[2 * c] += x.x;
        acc[2 * c + 1] += x.y;
      }
    }
  }
  uint4 v;
  v.x = pack_half2(acc[0], acc[1]);
  v.y = pack_half2(acc[2], acc[3]);
  v.z = pack_half2(acc[4], acc[5]);
  v.w = pack_half2(acc[6], acc[7]);
  reinterpret_cast<uint4*>(out)[idx] = v;
}

}  // namespace

int launch_combine(const float* o_accum, const float* lse_accum, void* o, float* lse, int64_t rows,
                   int num_splits, int h, int seqlen_q, int d, int64_t o_batch_stride,
                   int64_t o_row_stride, int64_t o_head_stride, cudaStream_t stream) {
  if (rows == 0) return FA_OK;
  const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (d == 128) {
    combine_kernel<128><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        o_accum, lse_accum, static_cast<__half*>(o), lse, rows, num_splits, h, seqlen_q,
        o_batch_stride, o_row_stride, o_head_stride);
  } else {
    combine_kernel<64><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        o_accum, lse_accum, static_cast<__half*>(o), lse, rows, num_splits, h, seqlen_q,
        o_batch_stride, o_row_stride, o_head_stride);
  }
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

}  // namespace fa

extern "C" int fa_combine(const FaCombineParams* p, fa_stream_t stream) {
  using namespace fa;
  FA_CHECK_ARG(p != nullptr, "fa_combine: params is NULL");
  FA_CHECK_ARG(p->o_accum && p->lse_accum && p->o, "fa_combine: o_accum, lse_accum, o must be non-NULL");
  if (p->d != 64 && p->d != 128)
    return set_error(FA_ERR_UNSUPPORTED, "fa_combine: head_dim must be 64 or 128");
  FA_CHECK_ARG(p->num_splits >= 1 && p->b >= 0 && p->h >= 1 && p->seqlen_q >= 0,
               "fa_combine: bad sizes");
  FA_CHECK_ARG(aligned16(p->o_accum) && (reinterpret_cast<uintptr_t>(p->o) & 7) == 0 &&
                   p->o_row_stride % 4 == 0 && p->o_head_stride % 4 == 0 && p->o_batch_stride % 4 == 0,
               "fa_combine: o_accum must be 16-byte aligned, o 8-byte aligned with strides multiple of 4");
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;
  const int64_t rows = static_cast<int64_t>(p->b) * p->h * p->seqlen_q;
  return launch_combine(p->o_accum, p->lse_accum, p->o, p->lse, rows, p->num_splits, p->h,
                        p->seqlen_q, p->d, p->o_batch_stride, p->o_row_stride, p->o_head_stride,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int fa_combine_gather(const FaCombineGatherParams* p, fa_stream_t stream) {
  using namespace fa;
  FA_CHECK_ARG(p != nullptr, "fa_combine_gather: params is NULL");
  FA_CHECK_ARG(p->num_parts >= 1 && p->num_parts <= FA_MAX_GATHER_PARTS, "fa_combine_gather: num_parts out of range");
  if (p->d != 64 && p->d != 128) return set_error(FA_ERR_UNSUPPORTED, "fa_combine_gather: head_dim must be 64 or 128");
  FA_CHECK_ARG(p->b >= 1 && p->h >= 1 && p->seqlen_q >= 1 && p->rows >= 0 && p->row_begin >= 0 &&
                   p->row_begin + p->rows <= p->seqlen_q,
               "fa_combine_gather: bad sizes");
  FA_CHECK_ARG(p->o && p->lse, "fa_combine_gather: o and lse must be non-NULL");
  GatherArgs a;
  for (int i = 0; i < FA_MAX_GATHER_PARTS; ++i) {
    a.o_part[i] = nullptr;
    a.lse_part[i] = nullptr;
  }
  for (int i = 0; i < p->num_parts; ++i) {
    FA_CHECK_ARG(p->o_part[i] && p->lse_part[i], "fa_combine_gather: NULL partial pointer");
    FA_CHECK_ARG(aligned16(p->o_part[i]), "fa_combine_gather: partials must be 16-byte aligned");
    a.o_part[i] = static_cast<const __half*>(p->o_part[i]);
    a.lse_part[i] = p->lse_part[i];
  }
  FA_CHECK_ARG(aligned16(p->o), "fa_combine_gather: o must be 16-byte aligned");
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;
  const int64_t total = static_cast<int64_t>(p->b) * p->rows * p->h;
  if (total == 0) return FA_OK;
  const int rows_per_block = kWarpsPerBlock * (32 / (p->d / 8));
  const unsigned blocks = static_cast<unsigned>((total + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->d == 128)
    combine_gather_kernel<128><<<blocks, kWarpsPerBlock * 32, 0, s>>>(a, static_cast<__half*>(p->o), p->lse, p->num_parts,
                                                                     p->b, p->h, p->seqlen_q, p->row_begin, p->rows);
  else
    combine_gather_kernel<64><<<blocks, kWarpsPerBlock * 32, 0, s>>>(a, static_cast<__half*>(p->o), p->lse, p->num_parts,
                                                                    p->b, p->h, p->seqlen_q, p->row_begin, p->rows);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}

extern "C" int fa_sum_gather(const FaSumGatherParams* p, fa_stream_t stream) {
  using namespace fa;
  FA_CHECK_ARG(p != nullptr, "fa_sum_gather: params is NULL");
  FA_CHECK_ARG(p->num_parts >= 1 && p->num_parts <= FA_MAX_GATHER_PARTS, "fa_sum_gather: num_parts out of range");
  if (p->d != 64 && p->d != 128) return set_error(FA_ERR_UNSUPPORTED, "fa_sum_gather: head_dim must be 64 or 128");
  FA_CHECK_ARG(p->b >= 1 && p->h >= 1 && p->seqlen_q >= 1 && p->rows >= 0 && p->row_begin >= 0 &&
                   p->row_begin + p->rows <= p->seqlen_q,
               "fa_sum_gather: bad sizes");
  FA_CHECK_ARG(p->out != nullptr && aligned16(p->out), "fa_sum_gather: out must be non-NULL and 16-byte aligned");
  SumArgs a;
  for (int i = 0; i < FA_MAX_GATHER_PARTS; ++i) {
    a.part[i] = nullptr;
    a.first_row[i] = 0;
  }
  for (int i = 0; i < p->num_parts; ++i) {
    FA_CHECK_ARG(p->part[i] != nullptr && aligned16(p->part[i]), "fa_sum_gather: parts must be non-NULL and 16-byte aligned");
    a.part[i] = static_cast<const __half*>(p->part[i]);
    a.first_row[i] = p->part_first_row[i];
  }
  int rc = check_device_sm100();
  if (rc != FA_OK) return rc;
  const int64_t vec_per_row = static_cast<int64_t>(p->h) * p->d / 8;
  const int64_t vec_per_slice = vec_per_row * p->rows;
  const int64_t total = vec_per_slice * p->b;
  if (total == 0) return FA_OK;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  sum_gather_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, static_cast<__half*>(p->out), p->num_parts, total, vec_per_slice, vec_per_row * p->seqlen_q,
      vec_per_row * p->row_begin, vec_per_row, p->row_begin);
  FA_CHECK_CUDA(cudaGetLastError());
  return FA_OK;
}
