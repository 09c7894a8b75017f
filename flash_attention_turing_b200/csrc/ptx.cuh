// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA
// (cp.async.bulk.tensor, no cluster multicast anywhere), tcgen05 MMA / TMEM, and the shared-memory /
// instruction descriptors of the 5th-generation tensor core.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

// ---------------------------------------------------------------------------------------------
// Device status word: kernels never trap.  A wait that runs out of time records a code here
// (first writer wins) and the CTA leaves through its normal exit path.
// ---------------------------------------------------------------------------------------------
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // bit 0: a bounded wait gave up; later CTAs return at once, outputs are invalid
  kStatusCapacityClamped = 2, // bit 1: a cache length exceeded the cache capacity and was clamped on the device
  kStatusSmemLayout = 4,      // bit 2: dynamic shared memory did not start on a 1024-byte boundary; the kernel did no work
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Non-blocking form (try_wait may suspend the thread for a while when the phase is incomplete).
__device__ __forceinline__ uint32_t mbar_test_nonblocking(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Per-CTA abort state shared by all waits of a kernel.
struct WaitCtx {
  volatile int* abort_flag;  // shared memory, 0 = running
  int* status;               // global status word (may be null)
  // Diagnosis of a wait that gave up: the FIRST one to do so also stores, in bits 8-31 of the status word,
  // `tag` (bits 8-15: which warp role waited) and the index of the barrier inside the kernel's barrier block
  // (bits 16-23; 8-byte units from `base`).  Both optional.
  int tag = 0;
  const void* base = nullptr;
  int iter = 0;  // loop iteration of the waiting role (bits 25-30), maintained by kernels that want it recorded
  uint64_t limit_ns = 4000000000ull;  // wall-clock limit of one wait
};

// The wait-timeout bit of the status word is sticky (until the host clears it): a CTA that starts while it is
// set does no work.  One thread reads the word and the answer is broadcast, so that the whole CTA takes the
// same way out even if the bit is set while the CTA starts.
// The same decision in two halves, for kernels that have a CTA-wide synchronisation early on anyway: thread 0
// starts reading the word at the top of the kernel and the value is consumed by a __syncthreads_or at that
// synchronisation, so the latency of the read overlaps the set-up instead of preceding it.
__device__ __forceinline__ int stop_probe_begin(const int* status) {
  return (threadIdx.x == 0 && status != nullptr) ? (*reinterpret_cast<const volatile int*>(status) & kStatusWaitTimeout) : 0;
}

__device__ __forceinline__ bool cta_should_stop(const int* status) {
  return __syncthreads_or(threadIdx.x == 0 && status != nullptr &&
                          (*reinterpret_cast<const volatile int*>(status) & kStatusWaitTimeout) != 0) != 0;
}

// Bounded wait on an mbarrier phase.  Returns false when the CTA is aborting (this wait or another
// one ran out of time); the caller must then fall through to the kernel's common exit.
// Limit: ctx.limit_ns of wall time measured with %globaltimer (4 s, far above any legitimate wait).
//
// Two forms, chosen per translation unit.  With FA_WAIT_INLINE the whole loop is inline at every wait (the
// backward kernels: with 96 registers per thread a call inside their loops costs spills, measured 5-25 %
// slower).  Without it, the bookkeeping that runs once per 1024 probes (abort flag, clock, time-out record) is
// one out-of-line function, and so is the spin of waits that are not on a critical path: inlined everywhere
// the loops made up a sixth of the forward kernel's code, which runs close to the capacity of the instruction
// cache (all warp roles execute different code at the same time; hit rate 82 % inline, 98 % out of line).
#ifdef FA_WAIT_INLINE
#ifdef FA_WAIT_SLIM
// Smallest inline form (the backward kernels: thirty waits each, and their code size is throughput -- 6 KB less
// code made them 2-6 % faster): the limit is a number of probes instead of wall time.  A probe of an incomplete
// phase suspends the thread for 3.96 us (measured), so 2^20 probes are about 4 s; only the role of the waiting
// warp is recorded with the time-out bit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_test(bar, parity)) return true;
  uint32_t spins = 0;
  while (true) {
    if (mbar_test(bar, parity)) return true;
    if (((++spins) & 0x3ff) == 0) {
      if (*ctx.abort_flag) return false;
      if (spins >= (1u << 20)) {
        *ctx.abort_flag = 1;
        if (ctx.status) atomicOr(ctx.status, kStatusWaitTimeout | ((ctx.tag & 0xff) << 8));
        return false;
      }
    }
  }
}
#else
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_test(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_test(bar, parity)) return true;
    if (((++spins) & 0x3ff) == 0) {
      if (*ctx.abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ctx.limit_ns) {
        *ctx.abort_flag = 1;
        if (ctx.status) {
          int idx = 0;
          if (ctx.base) idx = static_cast<int>((reinterpret_cast<const uint8_t*>(bar) - static_cast<const uint8_t*>(ctx.base)) >> 3) & 0xff;
          atomicCAS(ctx.status, 0, kStatusWaitTimeout | ((ctx.tag & 0xff) << 8) | (idx << 16) | ((parity & 1) << 24) | ((ctx.iter & 0x3f) << 25));
          atomicOr(ctx.status, kStatusWaitTimeout);
        }
        return false;
      }
    }
  }
}

#endif
__device__ __forceinline__ bool mbar_wait_hot(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  return mbar_wait(bar, parity, ctx);
}
#else
// `t0` is the time of the first check of this wait (0: this is the first); returns the value to pass next time,
// or 0 when the wait must be given up.
static __device__ __noinline__ uint64_t mbar_wait_check(uint64_t* bar, uint32_t parity, const WaitCtx* ctx,
                                                        uint64_t t0) {
  if (*ctx->abort_flag) return 0;
  const uint64_t now = global_timer_ns() | 1ull;
  if (t0 == 0) return now;
  if (now - t0 <= ctx->limit_ns) return t0;
  *ctx->abort_flag = 1;
  if (ctx->status) {
    int idx = 0;
    if (ctx->base) idx = static_cast<int>((reinterpret_cast<const uint8_t*>(bar) - static_cast<const uint8_t*>(ctx->base)) >> 3) & 0xff;
    atomicCAS(ctx->status, 0, kStatusWaitTimeout | ((ctx->tag & 0xff) << 8) | (idx << 16) | ((parity & 1) << 24) | ((ctx->iter & 0x3f) << 25));
    atomicOr(ctx->status, kStatusWaitTimeout);
  }
  return 0;
}

// For waits on a critical path: the spin is inline, so the waiter reacts within one probe of the barrier
// completing; only the bookkeeping is a call.
__device__ __forceinline__ bool mbar_wait_hot(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_test(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_test(bar, parity)) return true;
    if (((++spins) & 0x3ff) == 0) {
      t0 = mbar_wait_check(bar, parity, &ctx, t0);
      if (t0 == 0) return false;
    }
  }
}

// For all other waits: the first probe is inline, the whole spin a call (smallest code; the return from the call
// and the reloads after it cost the waiter some tens of clocks when the barrier completes).
static __device__ __noinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, const WaitCtx* ctx) {
  return mbar_wait_hot(bar, parity, *ctx);
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_test(bar, parity)) return true;
  return mbar_wait_spin(bar, parity, &ctx);
}
#endif

// Warp-collective form: every lane waits, and the warp agrees on the outcome so that it stays
// converged for the .sync.aligned instructions that follow.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  const bool ok = mbar_wait(bar, parity, ctx);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool mbar_wait_warp_hot(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  const bool ok = mbar_wait_hot(bar, parity, ctx);
  return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------------------------
// TMA: tiled bulk tensor loads global -> shared, completion on an mbarrier (tx bytes).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
        "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, ld/st, fences
// ---------------------------------------------------------------------------------------------
// Executed by one full warp.  Writes the TMEM base address to *smem_result.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// mbarrier arrive (count 1) once all tcgen05.mma issued so far by this thread have completed.
// Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]; A is a 128-lane fp16 tile packed two per 32-bit column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16 with fp16 A/B and fp32 D.
// bits [4,6) D format (1 = f32); [7,10) A format (0 = f16); [10,13) B format; bit 15 A major
// (0 = K-major, 1 = MN-major); bit 16 B major; [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, bool a_mn_major,
                                                      bool b_mn_major) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// Addresses and offsets are encoded in 16-byte units.
//   K-major operand  (rows x 64 fp16, one 128-byte row per matrix row, as TMA SWIZZLE_128B writes
//   it): SBO = 1024 B between 8-row groups, LBO unused.  Successive K=16 slices advance the start
//   address by 32 B.
//   MN-major operand (K rows of 64 contiguous MN elements = 128 B each): SBO = 1024 B between
//   8-row K groups, LBO = byte distance between consecutive 64-element MN chunks.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;  // descriptor version (Blackwell)
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// Cheap descriptor arithmetic for the MMA-issuing thread: the descriptor of a tile is built once, the
// descriptors of its K slices differ only in the start-address field (low word, 16-byte units).
__device__ __forceinline__ uint64_t desc_advance(uint64_t base, uint32_t byte_offset) {
  const uint32_t lo = static_cast<uint32_t>(base) + (byte_offset >> 4);
  return (base & 0xffffffff00000000ull) | lo;
}

// TMEM <-> registers, shape 32x32b: thread i of the warp owns lane (lane_base + i); xN = N
// consecutive 32-bit columns.  taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// Shape 16x256b: the warp touches 16 lanes starting at the lane field of taddr (0 or 16 inside its
// quarter).  With g = thread/4 and t = thread%4, repetition j gives r[4j], r[4j+1] = lane g, columns
// 8j+2t, 8j+2t+1 and r[4j+2], r[4j+3] = lane g+8, same columns: a row is spread over the four threads
// of a quad, so row reductions are two shuffles.  x8 = 64 columns.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}
// x4 = 32 columns: r[4j .. 4j+3] as above for j = 0..3.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
// Shape 16x128b: repetition j takes r[2j] -> lane g, column 4j+t and r[2j+1] -> lane g+8, column 4j+t:
// the layout of the 16x256b fragment after packing adjacent column pairs into one 32-bit word.
// x8 = 32 packed columns.
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                 "r"(r[7])
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// math helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed two-lane fp32 arithmetic and the three-input maximum of sm_100.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)),
        "l"(reinterpret_cast<uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float2 fsub2(float2 a, float2 b) {
  float2 d;
  asm("sub.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace fa
