/*
 * fa_b200.h -- C ABI of the B200 (sm_100a) FlashAttention launcher library `libfa_b200.so`.
 *
 * Every entry point takes plain pointers and sizes (no torch types), enqueues its kernels on the
 * stream it is given and returns without synchronising the host.  Return value: 0 on success, a
 * negative FA_ERR_* code otherwise; fa_last_error() returns the message of the calling thread's
 * last failure.  Invalid arguments are rejected on the host before any launch.  Unless stated
 * otherwise an entry point allocates nothing: outputs and scratch memory are owned by the caller.
 *
 * Each declaration names the reference interface it replaces (paths inside the reference project
 * Cy-47/flash-attention-turing).
 *
 * Tensor conventions: fp16 (IEEE half) data, fp32 log-sum-exp, int32 index arrays, all in device
 * memory.  Strides are in ELEMENTS and 64-bit; the innermost (head_dim) stride is always 1.
 * head_dim is 64 or 128.  Causal masking (is_causal = 1) is bottom-right aligned: key j is visible to query i
 * iff j <= i + seqlen_k - seqlen_q.  With is_causal = FA_CAUSAL_SHIFT (2) the diagonal is placed by the caller:
 * key j is visible to query i iff j <= i + causal_shift (dense layouts only) -- what a sequence-sharded run
 * needs to attend a block of query rows against a K/V shard in one launch.  A query row without a visible
 * key gets O = 0 and LSE = 0.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same underlying type as cudaStream_t (struct CUstream_st*); void* keeps the header CUDA-free. */
typedef void* fa_stream_t;

#define FA_CAUSAL_SHIFT 2 /* value of is_causal: the causal diagonal is given by causal_shift */

enum {
  FA_OK = 0,
  FA_ERR_INVALID_ARGUMENT = -1, /* shape / stride / pointer check failed on the host          */
  FA_ERR_UNSUPPORTED = -2,      /* head_dim not in {64,128}, wrong GPU architecture, ...       */
  FA_ERR_WORKSPACE = -3,        /* caller-provided scratch buffer is too small                 */
  FA_ERR_CUDA = -4              /* a CUDA runtime/driver call or the launch itself failed      */
};

/* Text of the calling thread's last error ("" if none). The pointer stays valid until the next
 * failing call on the same thread. */
const char* fa_last_error(void);

/* ABI version of this header; bumped on incompatible struct changes. */
int fa_abi_version(void);

/* Kernels never trap: every device-side wait (mbarrier, pipeline stage) is bounded, and a wait that
 * gives up records a non-zero code in a per-device status word and lets the kernel return.  This
 * call synchronises the current device and returns that word: 0 = no kernel reported a problem; bit 0
 * (value 1) = a wait timed out and the outputs of that launch are invalid; bit 1 (value 2) = a cache
 * length (cache_seqlens + seqlen_new, or seqused_k) exceeded the cache capacity and was clamped on the
 * device, so that a host that skips the reference's synchronising capacity check
 * (csrc/flash_attn/flash_api.cpp:627) still never reads or writes out of bounds; bit 2 (value 4) = the
 * dK/dV kernel found its dynamic shared memory not aligned to 1024 bytes (its head-size-128 layout has
 * no room for an alignment pad) and did no work, so dK and dV of that launch are invalid; negative =
 * FA_ERR_*.  With
 * reset != 0 the word is cleared afterwards.  Bit 0 is STICKY: while it is set, every later forward, backward
 * or decode launch on that device returns without doing any work (its outputs stay as they were) although the
 * host call reports FA_OK, until this function clears the word -- a host that wants to detect the condition
 * polls it.  When a wait gave up, bits 8-31 of the word identify the first one that did: bits 8-15 the warp
 * role that waited, bits 16-23 the index of the barrier in the kernel's barrier block, bit 24 the phase
 * parity, bits 25-30 the loop iteration (the backward kernels record the role only).  No counterpart in the
 * reference, whose launches are
 * not error-checked at all (src/flash_fwd_launch_template.h:73-89). */
int fa_device_status(int reset);

/* Self-test of the bounded waits: launches one tiny CTA that waits, with a limit of limit_us microseconds
 * (1 .. 1 000 000) instead of the kernels' 4 s, on a barrier nobody arrives on.  The wait gives up, bit 0 of
 * the status word is set (bits 8-15 read 0x7f), and the kernel returns normally: the path a real time-out
 * takes, without a hung launch.  Read and clear the word with fa_device_status(1) afterwards.  No
 * counterpart in the reference (its kernels have no bounded waits). */
int fa_selftest_wait_timeout(uint32_t limit_us, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* Forward: O = softmax(Q K^T * scale [+ causal mask]) V, LSE = logsumexp of the scaled scores.  */
/* Replaces mha_fwd / mha_varlen_fwd (csrc/flash_attn/flash_api.cpp:188-256, 353-416), the param */
/* struct Flash_fwd_params (csrc/flash_attn/src/flash.h:38-60), run_flash_fwd                    */
/* (src/flash_fwd_launch_template.h:49-93) and flash_fwd_kernel (src/flash_fwd_kernel.h:23-664). */
/* Also serves the tiled path of mha_fwd_kvcache (flash_api.cpp:686-714) through seqused_k,      */
/* cache_batch_idx and block_table, without the index_select copy the reference makes.           */
/* The kernel is persistent: one CTA per SM takes 256-row work items from a counter in device    */
/* memory (a pool of 1024 counter pairs inside the library; a launch takes the next pair and     */
/* leaves it zero), where the reference launches one CTA per row block of a max_seqlen-sized     */
/* grid (src/flash_fwd_launch_template.h:60-75).  Nothing for the host to manage: launches may   */
/* overlap on different streams and may be captured in CUDA graphs (first call on a device       */
/* outside the capture).  The dQ and dK/dV kernels of fa_bwd take their work the same way.       */
/* ------------------------------------------------------------------------------------------- */
typedef struct FaFwdParams {
  const void* q; /* dense (b, seqlen_q, h, d); varlen (total_q, h, d)                           */
  const void* k; /* dense (b_k, seqlen_k, h_k, d); varlen (total_k, h_k, d); paged (pages, page_size, h_k, d) */
  const void* v;
  void* o;       /* same layout family as q                                                    */
  float* lse;    /* (b, h, lse_row_stride) fp32, lse_row_stride >= seqlen_q                      */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t lse_row_stride;      /* elements between consecutive (b, h) rows of lse               */
  int32_t b;                   /* number of sequences                                           */
  int32_t seqlen_q, seqlen_k;  /* dense: exact; varlen: max_seqlen_q / max_seqlen_k             */
  int32_t h, h_k, d;
  int32_t total_q, total_k;    /* varlen only: rows of the packed q / k tensors                 */
  int32_t k_batch;             /* rows of dim 0 of k/v (cache batch or number of pages)         */
  float softmax_scale;
  int32_t is_causal;
  const int32_t* cu_seqlens_q; /* (b+1) or NULL (dense)                                         */
  const int32_t* cu_seqlens_k; /* (b+1) or NULL                                                 */
  const int32_t* seqused_k;    /* (b) keys actually used per sequence, or NULL                  */
  const int32_t* cache_batch_idx; /* (b) row of k/v dim 0 used by sequence i, or NULL           */
  const int32_t* block_table;  /* (b, block_table_batch_stride) page ids, or NULL               */
  int64_t block_table_batch_stride;
  int32_t page_size;           /* tokens per page (multiple of 128) when block_table != NULL    */
  int32_t block_table_cols;    /* columns of block_table (0 = unknown: seqused_k is trusted)    */
  int32_t causal_shift;        /* used when is_causal == FA_CAUSAL_SHIFT                        */
  int32_t reserved0;
} FaFwdParams;

int fa_fwd(const FaFwdParams* p, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* Backward: dQ, dK, dV from dO (and O, LSE of the forward).                                    */
/* Replaces mha_bwd / mha_varlen_bwd (flash_api.cpp:258-351, 418-506), Flash_bwd_params          */
/* (flash.h:62-83), run_flash_bwd (src/flash_bwd_launch_template.h:69-146) and its three kernels */
/* (flash_bwd_preprocess_kernel.h:23-96, flash_bwd_kernel.h:25-609 and :613-1344).  dK and dV    */
/* are written per KV head; the per-query-head buffers and the torch::sum_out reduction of the   */
/* reference (flash_api.cpp:338-348) do not exist here.                                          */
/* Two paths, chosen by `flags`:                                                                 */
/*   default (0)          a dQ kernel and a dK/dV kernel (seven products, like the reference's two  */
/*                        kernels); every result is bitwise reproducible run to run;               */
/*   FA_BWD_SINGLE_KERNEL ONE kernel with the five algorithmic products (S, dP, dV, dK, dQ); dQ is  */
/*                        accumulated in an fp32 scratch buffer with global reductions whose order */
/*                        depends on scheduling, so dQ is not bitwise reproducible (dK, dV are),  */
/*                        then converted to fp16 by a small pass.  Fewer tensor-core operations,  */
/*                        but the reductions cost the L2 cache more than the recomputation costs  */
/*                        the tensor cores: measured slower on B200 at every benchmark shape.     */
/* Scratch: `workspace` (256-byte aligned) must hold fa_bwd_workspace_bytes() bytes: fp32         */
/* rowsum(dO*O) and the LSE in base-2 units, and for FA_BWD_SINGLE_KERNEL the fp32 dQ accumulator */
/* (heads x padded rows x d).  The size depends on `flags`.                                      */
/* ------------------------------------------------------------------------------------------- */
#define FA_BWD_SINGLE_KERNEL 1
typedef struct FaBwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* dout;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  int64_t dq_batch_stride, dq_row_stride, dq_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t lse_row_stride;
  int32_t b, seqlen_q, seqlen_k, h, h_k, d;
  int32_t total_q, total_k;
  float softmax_scale;
  int32_t is_causal;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  void* workspace;
  size_t workspace_bytes;
  int32_t flags;      /* 0 or FA_BWD_SINGLE_KERNEL */
  int32_t causal_shift; /* used when is_causal == FA_CAUSAL_SHIFT */
} FaBwdParams;

size_t fa_bwd_workspace_bytes(const FaBwdParams* p);
int fa_bwd(const FaBwdParams* p, fa_stream_t stream);

/* Runs a subset of the launches of fa_bwd(): stage_mask bit 0 = preprocess (rowsum(dO*O), LSE in
 * base-2 units -> workspace; FA_BWD_SINGLE_KERNEL: also clears the dQ accumulator), bit 1 = the dQ kernel
 * (FA_BWD_SINGLE_KERNEL: the single backward kernel), bit 2 = the dK/dV kernel (FA_BWD_SINGLE_KERNEL: the
 * fp32 -> fp16 pass over dQ).  fa_bwd(p, s) is fa_bwd_stages(p, 7, s).  For timing one kernel at a time with CUDA events around the call (the
 * reference launches its three kernels back to back in run_flash_bwd,
 * src/flash_bwd_launch_template.h:84-138, and offers no such hook); bits 1 and 2 need a workspace that
 * an earlier call with bit 0 filled for the same inputs. */
int fa_bwd_stages(const FaBwdParams* p, int stage_mask, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* KV-cache step: append k_new/v_new in place at cache_seqlens, then attend q against            */
/* [0, cache_seqlens + seqlen_new) with split-KV and the LSE combine.                           */
/* Replaces mha_fwd_kvcache (flash_api.cpp:508-715), run_kvcache_paged_append /                  */
/* paged_append_kernel (src/kvcache_native.cu:782-871, 956-993), run_mha_fwd_kvcache_native      */
/* (:995-1218) with kvcache_decode_split_kernel / kvcache_split_kernel /                         */
/* kvcache_split_kernel_legacy (:148-674) and kvcache_combine_kernel (:676-780).                 */
/* No host synchronisation: the capacity check of the reference (flash_api.cpp:627) is the       */
/* caller's responsibility.  num_splits == 0 selects a split count from the shape                */
/* (choose_num_splits, kvcache_native.cu:913-952, retuned for 148 SMs).                          */
/* Scratch: fa_kvcache_workspace_bytes() bytes when the effective split count exceeds 1.         */
/* ------------------------------------------------------------------------------------------- */
typedef struct FaKvcacheParams {
  const void* q;       /* (b, seqlen_q, h, d)                                                   */
  void* k_cache;       /* contiguous (b_cache, seqlen_cache, h_k, d) or paged (pages, page_size, h_k, d) */
  void* v_cache;
  const void* k_new;   /* (b, seqlen_new, h_k, d) or NULL                                        */
  const void* v_new;
  void* o;             /* (b, seqlen_q, h, d)                                                   */
  float* lse;          /* (b, h, seqlen_q)                                                      */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t kc_batch_stride, kc_row_stride, kc_head_stride;
  int64_t vc_batch_stride, vc_row_stride, vc_head_stride;
  int64_t kn_batch_stride, kn_row_stride, kn_head_stride;
  int64_t vn_batch_stride, vn_row_stride, vn_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int32_t b, seqlen_q, seqlen_new, h, h_k, d;
  int32_t cache_batch;         /* dim 0 of the cache tensors (cache rows or pages)              */
  int32_t seqlen_cache;        /* dim 1 of the cache tensors (capacity per row, or page size)   */
  float softmax_scale;
  int32_t is_causal;
  const int32_t* cache_seqlens;    /* (b) tokens in the cache BEFORE the append                 */
  const int32_t* cache_batch_idx;  /* (b) or NULL; contiguous cache only                        */
  const int32_t* block_table;      /* (b, block_table_batch_stride) or NULL                     */
  int64_t block_table_batch_stride;
  int32_t max_blocks_per_seq;      /* columns of block_table                                    */
  int32_t num_splits;              /* 0 = heuristic                                             */
  void* workspace;
  size_t workspace_bytes;
} FaKvcacheParams;

/* Split count fa_kvcache() will use for these parameters (resolves num_splits == 0). */
int fa_kvcache_num_splits(const FaKvcacheParams* p);
size_t fa_kvcache_workspace_bytes(const FaKvcacheParams* p);
int fa_kvcache(const FaKvcacheParams* p, fa_stream_t stream);

/* KV-cache step for hosts that cannot allocate device memory.  No counterpart in the reference.   */
/*                                                                                             */
/* Some callers of this library have no allocator to hand the split-KV scratch from: a serving    */
/* loop whose memory pool was sized and frozen at start-up, a plugin running inside another       */
/* runtime's stream callback or graph node where cudaMalloc is forbidden, a host written in a     */
/* language binding that exposes launches but not allocation.  fa_kvcache_noalloc() does what      */
/* fa_kvcache() does, with identical kernels and results, but takes the partial (O, LSE) scratch   */
/* from an array that is part of the library image itself; p->workspace and p->workspace_bytes are */
/* ignored.  It calls no cudaMalloc / cudaFree and no allocating library routine.                 */
/*                                                                                             */
/* Limit: the array is FA_KVCACHE_NOALLOC_SCRATCH_BYTES (32 MiB) per GPU, held by every GPU that  */
/* loads the library until the process exits.  A call that needs more -- i.e. whose               */
/* fa_kvcache_workspace_bytes() exceeds that -- is rejected with FA_ERR_WORKSPACE and nothing is  */
/* launched (use fewer splits, or fa_kvcache() with your own buffer).                             */
/* First call on a device: the library looks up the device address of the array (one              */
/* cudaGetSymbolAddress with that device current) and caches it; make this first call outside any */
/* stream capture.                                                                             */
/* Sharing: every call on a GPU uses the same array.  The kernels overwrite every element they     */
/* later read, so no clearing is needed between calls, but two calls that can overlap on the GPU   */
/* (different streams without an ordering between them) race on it: serialise them.               */
/* ------------------------------------------------------------------------------------------- */
#define FA_KVCACHE_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)
int fa_kvcache_noalloc(const FaKvcacheParams* p, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* Stand-alone log-sum-exp merge of split partials:                                             */
/*   LSE = logsumexp_s lse_accum[s], O = sum_s exp(lse_accum[s] - LSE) * o_accum[s].            */
/* Replaces kvcache_combine_kernel / kvcache_combine_kernel_legacy (kvcache_native.cu:676-780).  */
/* Also the local step after the (O, LSE) exchange of a sequence-sharded forward.               */
/* o_accum: (num_splits, rows, d) fp32; lse_accum: (num_splits, rows) fp32, -inf for an empty    */
/* split; rows are ordered (b, h, seqlen_q).  Rows whose every split is empty get O=0, LSE=0.    */
/* ------------------------------------------------------------------------------------------- */
typedef struct FaCombineParams {
  const float* o_accum;
  const float* lse_accum;
  void* o;          /* fp16 (b, seqlen_q, h, d) through the strides below                       */
  float* lse;       /* (b, h, seqlen_q) contiguous, or NULL                                      */
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int32_t num_splits, b, h, seqlen_q, d;
  int32_t reserved0;
} FaCombineParams;

int fa_combine(const FaCombineParams* p, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* Merge of per-rank partial results of a sequence-sharded forward, reading the partials where    */
/* they are: o_part[r] / lse_part[r] may point into ANOTHER GPU's memory (peer-mapped, e.g. a    */
/* symmetric-memory buffer); the kernel reads them with ordinary loads over NVLink, so the        */
/* exchange and the merge are one kernel and no staging copy or all-to-all is needed.  No         */
/* counterpart in the reference (it has no multi-GPU code); the arithmetic is that of              */
/* kvcache_combine_kernel (kvcache_native.cu:676-729).                                           */
/* Partials are in the layout the forward writes: o_part[r] fp16 (b, seqlen_q, h, d) contiguous,  */
/* lse_part[r] fp32 (b, h, seqlen_q) contiguous, -inf where rank r saw no key.  This call merges  */
/* query rows [row_begin, row_begin + rows) of every sequence into o (b, rows, h, d) fp16 and     */
/* lse (b, h, rows) fp32.  The caller orders the call after every rank has finished its partial.   */
/* o and every o_part[r] must be 16-byte aligned.                                                   */
/* ------------------------------------------------------------------------------------------- */
#define FA_MAX_GATHER_PARTS 16
typedef struct FaCombineGatherParams {
  const void* o_part[FA_MAX_GATHER_PARTS];
  const float* lse_part[FA_MAX_GATHER_PARTS];
  void* o;
  float* lse;
  int32_t num_parts, b, h, seqlen_q, d;
  int32_t row_begin, rows;
  int32_t reserved0;
} FaCombineGatherParams;

int fa_combine_gather(const FaCombineGatherParams* p, fa_stream_t stream);

/* ------------------------------------------------------------------------------------------- */
/* Sum of per-rank partial gradients of a sequence-sharded backward, read where they are: with   */
/* K/V sharded by sequence every rank computes dK/dV of its own shard completely, but only its   */
/* keys' share of dQ; the shares add up.  part[r] is rank r's fp16 dQ share for ALL query rows,   */
/* (b, seqlen_q, h, d) contiguous, and may point into another GPU's memory (peer-mapped, plain   */
/* loads over NVLink).  This call adds rows [row_begin, row_begin + rows) of every part in fp32   */
/* and writes out (b, rows, h, d) fp16 -- exchange and reduction in one kernel.  No counterpart  */
/* in the reference (it has no multi-GPU code; its only cross-CTA gradient sum is the GQA        */
/* torch::sum_out of flash_api.cpp:338-348).                                                     */
/* ------------------------------------------------------------------------------------------- */
typedef struct FaSumGatherParams {
  const void* part[FA_MAX_GATHER_PARTS];
  void* out;
  int32_t num_parts, b, h, seqlen_q, d;
  int32_t row_begin, rows;
  int32_t reserved0;
  /* part_first_row[r]: query rows below this index hold nothing in part r (a causal shard sees no key    */
  /* there) and are neither read nor added; 0 = every row is valid.                                      */
  int32_t part_first_row[FA_MAX_GATHER_PARTS];
} FaSumGatherParams;

int fa_sum_gather(const FaSumGatherParams* p, fa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
