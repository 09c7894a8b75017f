// PyTorch binding of libfa_b200.so: the five functions the reference extension exports
// (PYBIND11_MODULE in csrc/flash_attn/flash_api.cpp:717-724) with the same names, argument order
// and checks.  This file only validates tensors, allocates outputs and scratch memory with the
// torch caching allocator, fills the C-ABI parameter structs and calls the launcher on the current
// CUDA stream of q's device.  It contains no kernels and has no CPU path.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "../../include/fa_b200.h"

namespace {

int g_bwd_flags = 0;  // flags of FaBwdParams used by bwd / varlen_bwd (set_single_kernel_backward)


void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == FA_OK, what, " failed (", rc, "): ", fa_last_error());
}

void check_supported_head_dim(int64_t d) {
  // message of check_supported_head_dim, flash_api.cpp:10-14
  TORCH_CHECK(d == 64 || d == 128, "Turing FlashAttention supports head_dim 64 or 128");
}

void check_half_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kHalf, name, " must be a float16 tensor");
  TORCH_CHECK(t.stride(-1) == 1, name, " must have contiguous last dimension");
}

fa_stream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// A log-sum-exp tensor (b, h, rows) given by the caller: fp32, unit stride along rows, heads of a batch one
// row pitch apart -- e.g. a slice of the rows of a contiguous tensor.
void check_lse_view(const at::Tensor& l, int64_t b, int64_t h, int64_t rows, const char* name) {
  TORCH_CHECK(l.is_cuda() && l.scalar_type() == torch::kFloat32 && l.dim() == 3, name,
              " must be a float32 CUDA tensor of rank 3");
  TORCH_CHECK(l.size(0) == b && l.size(1) == h && l.size(2) == rows, name,
              " must have shape [batch_size, nheads_q, seqlen_q]");
  TORCH_CHECK((rows == 1 || l.stride(2) == 1) && l.stride(1) >= rows && (b == 1 || l.stride(0) == h * l.stride(1)), name,
              " must have unit stride along the rows and batches h row pitches apart");
}

// ---- dense forward (mha_fwd, flash_api.cpp:188-256) ----
// out_, lse_ (optional, after the reference's five arguments): write O and LSE there instead of into new tensors
// (strided views are fine: e.g. a block of rows of a larger buffer).  causal_shift_ (optional): with is_causal,
// key j is visible to query i iff j <= i + causal_shift instead of the bottom-right alignment.
std::vector<at::Tensor> mha_fwd(at::Tensor q, at::Tensor k, at::Tensor v, const double softmax_scale,
                                bool is_causal, c10::optional<at::Tensor> out_, c10::optional<at::Tensor> lse_,
                                c10::optional<int64_t> causal_shift_) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be rank-4 tensors");
  check_half_cuda(q, "q");
  check_half_cuda(k, "k");
  check_half_cuda(v, "v");
  const int64_t batch_size = q.size(0), seqlen_q = q.size(1), num_heads = q.size(2), head_size = q.size(3);
  const int64_t seqlen_k = k.size(1), num_heads_k = k.size(2);
  TORCH_CHECK(k.size(0) == batch_size && v.size(0) == batch_size, "k/v batch size must match q");
  TORCH_CHECK(v.size(1) == seqlen_k, "k and v seqlen_k must match");
  TORCH_CHECK(v.size(2) == num_heads_k, "k and v num_heads must match");
  TORCH_CHECK(k.size(3) == head_size && v.size(3) == head_size, "q/k/v head_dim must match");
  TORCH_CHECK(num_heads % num_heads_k == 0, "num_heads_q must be divisible by num_heads_k for GQA/MQA");
  check_supported_head_dim(head_size);
  c10::cuda::CUDAGuard guard(q.device());

  at::Tensor o = (out_.has_value() && out_->defined()) ? *out_ : torch::empty(q.sizes(), q.options());
  at::Tensor l = (lse_.has_value() && lse_->defined())
                     ? *lse_ : torch::empty({batch_size, num_heads, seqlen_q}, q.options().dtype(torch::kFloat32));
  if (out_.has_value() && out_->defined()) {
    check_half_cuda(o, "out");
    TORCH_CHECK(o.sizes() == q.sizes() && o.device() == q.device(), "out must have the shape and device of q");
  }
  if (lse_.has_value() && lse_->defined()) check_lse_view(l, batch_size, num_heads, seqlen_q, "lse");
  if (batch_size == 0 || seqlen_q == 0) return {o, l};
  if (seqlen_k == 0) {
    o.zero_();
    l.zero_();
    return {o, l};
  }

  FaFwdParams p = {};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.o = o.data_ptr();
  p.lse = l.data_ptr<float>();
  p.q_batch_stride = q.stride(0); p.q_row_stride = q.stride(1); p.q_head_stride = q.stride(2);
  p.k_batch_stride = k.stride(0); p.k_row_stride = k.stride(1); p.k_head_stride = k.stride(2);
  p.v_batch_stride = v.stride(0); p.v_row_stride = v.stride(1); p.v_head_stride = v.stride(2);
  p.o_batch_stride = o.stride(0); p.o_row_stride = o.stride(1); p.o_head_stride = o.stride(2);
  p.lse_row_stride = l.stride(1);
  p.b = batch_size; p.seqlen_q = seqlen_q; p.seqlen_k = seqlen_k;
  p.h = num_heads; p.h_k = num_heads_k; p.d = head_size;
  p.k_batch = batch_size;
  p.softmax_scale = static_cast<float>(softmax_scale);
  p.is_causal = is_causal;
  if (is_causal && causal_shift_.has_value()) {
    p.is_causal = FA_CAUSAL_SHIFT;
    p.causal_shift = static_cast<int32_t>(*causal_shift_);
  }
  check_rc(fa_fwd(&p, current_stream()), "fa_fwd");
  return {o, l};
}

void check_cu_seqlens(const at::Tensor& cu_seqlens_q, const at::Tensor& cu_seqlens_k) {
  TORCH_CHECK(cu_seqlens_q.is_cuda() && cu_seqlens_k.is_cuda(), "cu_seqlens_q/cu_seqlens_k must be CUDA tensors");
  TORCH_CHECK(cu_seqlens_q.scalar_type() == torch::kInt32 && cu_seqlens_k.scalar_type() == torch::kInt32,
              "cu_seqlens_q/cu_seqlens_k must be int32 tensors");
  TORCH_CHECK(cu_seqlens_q.is_contiguous() && cu_seqlens_k.is_contiguous(),
              "cu_seqlens_q/cu_seqlens_k must be contiguous");
  TORCH_CHECK(cu_seqlens_q.dim() == 1 && cu_seqlens_k.dim() == 1, "cu_seqlens_q/cu_seqlens_k must be rank-1");
  TORCH_CHECK(cu_seqlens_q.numel() >= 2 && cu_seqlens_k.numel() >= 2,
              "cu_seqlens_q/cu_seqlens_k must have at least 2 elements");
  TORCH_CHECK(cu_seqlens_k.numel() == cu_seqlens_q.numel(),
              "cu_seqlens_k must have shape [batch_size + 1] with cumulative offsets");
}

void check_varlen_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be rank-3 packed tensors");
  check_half_cuda(q, "q");
  check_half_cuda(k, "k");
  check_half_cuda(v, "v");
  TORCH_CHECK(k.size(0) == v.size(0), "k and v total tokens must match");
  TORCH_CHECK(k.size(1) == v.size(1), "k and v num_heads must match");
  TORCH_CHECK(k.size(2) == v.size(2), "k and v head_dim must match");
  TORCH_CHECK(q.size(2) == k.size(2), "q/k/v head_dim must match");
  TORCH_CHECK(q.size(1) % k.size(1) == 0, "num_heads_q must be divisible by num_heads_k for GQA/MQA");
  check_supported_head_dim(q.size(2));
}

// ---- varlen forward (mha_varlen_fwd, flash_api.cpp:353-416) ----
std::vector<at::Tensor> mha_varlen_fwd(at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor cu_seqlens_q,
                                       at::Tensor cu_seqlens_k, const int64_t max_seqlen_q,
                                       const int64_t max_seqlen_k, const double softmax_scale,
                                       bool is_causal) {
  check_varlen_qkv(q, k, v);
  check_cu_seqlens(cu_seqlens_q, cu_seqlens_k);
  const int64_t batch_size = cu_seqlens_q.numel() - 1;
  const int64_t num_heads = q.size(1), num_heads_k = k.size(1), head_size = q.size(2);
  c10::cuda::CUDAGuard guard(q.device());

  at::Tensor out = torch::zeros_like(q);  // rows outside every sequence stay zero, as in the reference
  at::Tensor l = torch::zeros({batch_size, num_heads, max_seqlen_q}, q.options().dtype(torch::kFloat32));
  if (q.size(0) == 0 || k.size(0) == 0 || max_seqlen_q <= 0) return {out, l};

  FaFwdParams p = {};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.o = out.data_ptr();
  p.lse = l.data_ptr<float>();
  p.q_row_stride = q.stride(0); p.q_head_stride = q.stride(1); p.q_batch_stride = 0;
  p.k_row_stride = k.stride(0); p.k_head_stride = k.stride(1); p.k_batch_stride = 0;
  p.v_row_stride = v.stride(0); p.v_head_stride = v.stride(1); p.v_batch_stride = 0;
  p.o_row_stride = out.stride(0); p.o_head_stride = out.stride(1); p.o_batch_stride = 0;
  p.lse_row_stride = max_seqlen_q;
  p.b = batch_size; p.seqlen_q = max_seqlen_q; p.seqlen_k = max_seqlen_k;
  p.h = num_heads; p.h_k = num_heads_k; p.d = head_size;
  p.total_q = q.size(0); p.total_k = k.size(0);
  p.softmax_scale = static_cast<float>(softmax_scale);
  p.is_causal = is_causal;
  p.cu_seqlens_q = cu_seqlens_q.data_ptr<int>();
  p.cu_seqlens_k = cu_seqlens_k.data_ptr<int>();
  check_rc(fa_fwd(&p, current_stream()), "fa_fwd");
  return {out, l};
}

// ---- dense backward (mha_bwd, flash_api.cpp:258-351) ----
// Gradient destination given by the caller (e.g. a view into a packed dqkv tensor) or allocated here.
at::Tensor grad_destination(const c10::optional<at::Tensor>& given, const at::Tensor& like, const char* name,
                            bool zero_init) {
  if (!given.has_value() || !given->defined())
    return zero_init ? torch::zeros_like(like, like.options(), at::MemoryFormat::Contiguous)
                     : torch::empty_like(like, like.options(), at::MemoryFormat::Contiguous);
  const at::Tensor& g = *given;
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == torch::kFloat16 && g.device() == like.device(), name,
              " must be a float16 CUDA tensor on the device of its input");
  TORCH_CHECK(g.sizes() == like.sizes(), name, " must have the shape of its input");
  TORCH_CHECK(g.stride(-1) == 1, name, " must have a contiguous last dimension");
  if (zero_init) g.zero_();
  return g;
}

// dq_, dk_, dv_ (optional, after the reference's eight arguments): write the gradients there instead of
// into new tensors; strided views are fine (16-byte aligned, strides multiples of 8 elements).
std::vector<at::Tensor> mha_bwd(at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor out, at::Tensor l,
                                at::Tensor dout, const double softmax_scale, bool is_causal,
                                c10::optional<at::Tensor> dq_, c10::optional<at::Tensor> dk_,
                                c10::optional<at::Tensor> dv_, c10::optional<int64_t> causal_shift_) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be rank-4 tensors");
  TORCH_CHECK(out.dim() == 4 && dout.dim() == 4, "out and dout must be rank-4 tensors");
  check_half_cuda(q, "q"); check_half_cuda(k, "k"); check_half_cuda(v, "v");
  check_half_cuda(out, "out"); check_half_cuda(dout, "dout");
  const int64_t batch_size = q.size(0), seqlen_q = q.size(1), num_heads = q.size(2), head_size = q.size(3);
  const int64_t seqlen_k = k.size(1), num_heads_k = k.size(2);
  TORCH_CHECK(k.size(0) == batch_size && v.size(0) == batch_size, "k/v batch size must match q");
  TORCH_CHECK(v.size(1) == seqlen_k, "k and v seqlen_k must match");
  TORCH_CHECK(v.size(2) == num_heads_k, "k and v num_heads must match");
  TORCH_CHECK(k.size(3) == head_size && v.size(3) == head_size, "q/k/v head_dim must match");
  TORCH_CHECK(out.sizes() == q.sizes() && dout.sizes() == q.sizes(), "out and dout must match q shape");
  TORCH_CHECK(num_heads % num_heads_k == 0, "num_heads_q must be divisible by num_heads_k for GQA/MQA");
  check_supported_head_dim(head_size);
  check_lse_view(l, batch_size, num_heads, seqlen_q, "l");
  c10::cuda::CUDAGuard guard(q.device());

  at::Tensor dq = grad_destination(dq_, q, "dq", false);
  at::Tensor dk = grad_destination(dk_, k, "dk", false);
  at::Tensor dv = grad_destination(dv_, v, "dv", false);
  if (batch_size == 0 || seqlen_q == 0 || seqlen_k == 0) {
    dq.zero_(); dk.zero_(); dv.zero_();
    return {dq, dk, dv};
  }

  FaBwdParams p = {};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.o = out.data_ptr();
  p.dout = dout.data_ptr(); p.lse = l.data_ptr<float>();
  p.dq = dq.data_ptr(); p.dk = dk.data_ptr(); p.dv = dv.data_ptr();
  p.q_batch_stride = q.stride(0); p.q_row_stride = q.stride(1); p.q_head_stride = q.stride(2);
  p.k_batch_stride = k.stride(0); p.k_row_stride = k.stride(1); p.k_head_stride = k.stride(2);
  p.v_batch_stride = v.stride(0); p.v_row_stride = v.stride(1); p.v_head_stride = v.stride(2);
  p.o_batch_stride = out.stride(0); p.o_row_stride = out.stride(1); p.o_head_stride = out.stride(2);
  p.do_batch_stride = dout.stride(0); p.do_row_stride = dout.stride(1); p.do_head_stride = dout.stride(2);
  p.dq_batch_stride = dq.stride(0); p.dq_row_stride = dq.stride(1); p.dq_head_stride = dq.stride(2);
  p.dk_batch_stride = dk.stride(0); p.dk_row_stride = dk.stride(1); p.dk_head_stride = dk.stride(2);
  p.dv_batch_stride = dv.stride(0); p.dv_row_stride = dv.stride(1); p.dv_head_stride = dv.stride(2);
  p.lse_row_stride = l.stride(1);
  p.b = batch_size; p.seqlen_q = seqlen_q; p.seqlen_k = seqlen_k;
  p.h = num_heads; p.h_k = num_heads_k; p.d = head_size;
  p.softmax_scale = static_cast<float>(softmax_scale);
  p.is_causal = is_causal;
  if (is_causal && causal_shift_.has_value()) {
    p.is_causal = FA_CAUSAL_SHIFT;
    p.causal_shift = static_cast<int32_t>(*causal_shift_);
  }
  p.flags = g_bwd_flags;
  const size_t ws = fa_bwd_workspace_bytes(&p);
  at::Tensor workspace = torch::empty({static_cast<int64_t>(ws)}, q.options().dtype(torch::kUInt8));
  p.workspace = workspace.data_ptr();
  p.workspace_bytes = ws;
  check_rc(fa_bwd(&p, current_stream()), "fa_bwd");
  return {dq, dk, dv};
}

// ---- varlen backward (mha_varlen_bwd, flash_api.cpp:418-506) ----
std::vector<at::Tensor> mha_varlen_bwd(at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor out, at::Tensor l,
                                       at::Tensor dout, at::Tensor cu_seqlens_q, at::Tensor cu_seqlens_k,
                                       const int64_t max_seqlen_q, const int64_t max_seqlen_k,
                                       const double softmax_scale, bool is_causal,
                                       c10::optional<at::Tensor> dq_, c10::optional<at::Tensor> dk_,
                                       c10::optional<at::Tensor> dv_) {
  check_varlen_qkv(q, k, v);
  check_cu_seqlens(cu_seqlens_q, cu_seqlens_k);
  check_half_cuda(out, "out");
  check_half_cuda(dout, "dout");
  TORCH_CHECK(out.sizes() == q.sizes(), "out must match q shape");
  TORCH_CHECK(dout.sizes() == q.sizes(), "dout must match q shape");
  TORCH_CHECK(l.dim() == 3, "l must be rank-3 for varlen_bwd");
  const int64_t batch_size = cu_seqlens_q.numel() - 1;
  const int64_t num_heads = q.size(1), num_heads_k = k.size(1), head_size = q.size(2);
  TORCH_CHECK(l.size(0) == batch_size && l.size(1) == num_heads && l.size(2) == max_seqlen_q,
              "l must have shape [batch_size, nheads_q, max_seqlen_q]");
  TORCH_CHECK(l.is_cuda() && l.scalar_type() == torch::kFloat32 && l.is_contiguous(),
              "l must be a contiguous float32 CUDA tensor");
  c10::cuda::CUDAGuard guard(q.device());

  // rows outside every sequence stay zero, as in the reference (torch::zeros_like, :462-464)
  at::Tensor dq = grad_destination(dq_, q, "dq", true);
  at::Tensor dk = grad_destination(dk_, k, "dk", true);
  at::Tensor dv = grad_destination(dv_, v, "dv", true);
  if (q.size(0) == 0 || k.size(0) == 0 || max_seqlen_q <= 0 || max_seqlen_k <= 0) return {dq, dk, dv};

  FaBwdParams p = {};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.o = out.data_ptr();
  p.dout = dout.data_ptr(); p.lse = l.data_ptr<float>();
  p.dq = dq.data_ptr(); p.dk = dk.data_ptr(); p.dv = dv.data_ptr();
  p.q_row_stride = q.stride(0); p.q_head_stride = q.stride(1);
  p.k_row_stride = k.stride(0); p.k_head_stride = k.stride(1);
  p.v_row_stride = v.stride(0); p.v_head_stride = v.stride(1);
  p.o_row_stride = out.stride(0); p.o_head_stride = out.stride(1);
  p.do_row_stride = dout.stride(0); p.do_head_stride = dout.stride(1);
  p.dq_row_stride = dq.stride(0); p.dq_head_stride = dq.stride(1);
  p.dk_row_stride = dk.stride(0); p.dk_head_stride = dk.stride(1);
  p.dv_row_stride = dv.stride(0); p.dv_head_stride = dv.stride(1);
  p.lse_row_stride = max_seqlen_q;
  p.b = batch_size; p.seqlen_q = max_seqlen_q; p.seqlen_k = max_seqlen_k;
  p.h = num_heads; p.h_k = num_heads_k; p.d = head_size;
  p.total_q = q.size(0); p.total_k = k.size(0);
  p.softmax_scale = static_cast<float>(softmax_scale);
  p.is_causal = is_causal;
  p.cu_seqlens_q = cu_seqlens_q.data_ptr<int>();
  p.cu_seqlens_k = cu_seqlens_k.data_ptr<int>();
  p.flags = g_bwd_flags;
  const size_t ws = fa_bwd_workspace_bytes(&p);
  at::Tensor workspace = torch::empty({static_cast<int64_t>(ws)}, q.options().dtype(torch::kUInt8));
  p.workspace = workspace.data_ptr();
  p.workspace_bytes = ws;
  check_rc(fa_bwd(&p, current_stream()), "fa_bwd");
  return {dq, dk, dv};
}

// ---- KV-cache forward (mha_fwd_kvcache, flash_api.cpp:508-715) ----
std::vector<at::Tensor> mha_fwd_kvcache(at::Tensor q, at::Tensor k_cache, at::Tensor v_cache, py::object k_obj,
                                        py::object v_obj, at::Tensor cache_seqlens, py::object rotary_cos_obj,
                                        py::object rotary_sin_obj, py::object cache_batch_idx_obj,
                                        py::object cache_leftpad_obj, py::object block_table_obj,
                                        py::object alibi_slopes_obj, py::object out_obj,
                                        const double softmax_scale, bool is_causal, int64_t window_size_left,
                                        int64_t window_size_right, const double softcap,
                                        bool rotary_interleaved, int64_t num_splits) {
  (void)rotary_interleaved;
  TORCH_CHECK(rotary_cos_obj.is_none() && rotary_sin_obj.is_none(),
              "Turing KV-cache does not support rotary embeddings yet");
  TORCH_CHECK(cache_leftpad_obj.is_none(), "Turing KV-cache does not support cache_leftpad yet");
  TORCH_CHECK(alibi_slopes_obj.is_none(), "Turing KV-cache does not support ALiBi yet");
  TORCH_CHECK(out_obj.is_none(), "Turing KV-cache does not support a preallocated output tensor yet");
  TORCH_CHECK(window_size_left == -1 && window_size_right == -1,
              "Turing KV-cache does not support local window attention yet");
  TORCH_CHECK(softcap == 0.0, "Turing KV-cache does not support softcap yet");
  TORCH_CHECK(num_splits >= 0, "num_splits must be non-negative");

  TORCH_CHECK(q.is_cuda() && k_cache.is_cuda() && v_cache.is_cuda(), "q, k_cache, v_cache must be CUDA tensors");
  TORCH_CHECK(q.scalar_type() == torch::kFloat16 && k_cache.scalar_type() == torch::kFloat16 &&
                  v_cache.scalar_type() == torch::kFloat16,
              "q, k_cache, v_cache must be float16 tensors");
  TORCH_CHECK(q.dim() == 4 && k_cache.dim() == 4 && v_cache.dim() == 4,
              "q, k_cache, v_cache must be rank-4 tensors");
  TORCH_CHECK(k_cache.size(1) == v_cache.size(1), "k_cache and v_cache seqlen must match");
  TORCH_CHECK(k_cache.size(2) == v_cache.size(2), "k_cache and v_cache num_heads must match");
  TORCH_CHECK(q.size(3) == k_cache.size(3) && q.size(3) == v_cache.size(3),
              "q, k_cache, v_cache head_dim must match");
  TORCH_CHECK(q.size(2) % k_cache.size(2) == 0, "num_heads_q must be divisible by num_heads_k for GQA/MQA");
  check_supported_head_dim(q.size(3));
  TORCH_CHECK(q.stride(-1) == 1 && k_cache.stride(-1) == 1 && v_cache.stride(-1) == 1,
              "q, k_cache, v_cache must have contiguous last dimension");
  TORCH_CHECK(cache_seqlens.is_cuda(), "cache_seqlens must be a CUDA tensor");
  TORCH_CHECK(cache_seqlens.scalar_type() == torch::kInt32, "cache_seqlens must be an int32 tensor");
  TORCH_CHECK(cache_seqlens.is_contiguous(), "cache_seqlens must be contiguous");
  TORCH_CHECK(cache_seqlens.dim() == 1 && cache_seqlens.numel() == q.size(0),
              "cache_seqlens must have shape [batch_size]");

  const int64_t batch_size = q.size(0), seqlen_q = q.size(1), num_heads = q.size(2), head_size = q.size(3);
  const int64_t num_heads_k = k_cache.size(2);
  const bool has_block_table = !block_table_obj.is_none();
  at::Tensor block_table;
  int64_t batch_size_cache = k_cache.size(0);
  if (has_block_table) {
    block_table = block_table_obj.cast<at::Tensor>();
    TORCH_CHECK(block_table.is_cuda(), "block_table must be a CUDA tensor");
    TORCH_CHECK(block_table.scalar_type() == torch::kInt32, "block_table must be an int32 tensor");
    TORCH_CHECK(block_table.stride(-1) == 1, "block_table must have contiguous last dimension");
    TORCH_CHECK(block_table.dim() == 2 && block_table.size(0) == batch_size,
                "block_table must have shape [batch_size, max_num_blocks_per_seq]");
    TORCH_CHECK(k_cache.size(1) % 256 == 0, "Paged KV cache block size must be divisible by 256");
    batch_size_cache = batch_size;
  }

  at::Tensor cache_batch_idx;
  const bool has_cache_batch_idx = !cache_batch_idx_obj.is_none();
  if (has_cache_batch_idx) {
    TORCH_CHECK(!has_block_table, "Paged KV cache does not support cache_batch_idx");
    cache_batch_idx = cache_batch_idx_obj.cast<at::Tensor>();
    TORCH_CHECK(cache_batch_idx.is_cuda(), "cache_batch_idx must be a CUDA tensor");
    TORCH_CHECK(cache_batch_idx.scalar_type() == torch::kInt32, "cache_batch_idx must be an int32 tensor");
    TORCH_CHECK(cache_batch_idx.is_contiguous(), "cache_batch_idx must be contiguous");
    TORCH_CHECK(cache_batch_idx.dim() == 1 && cache_batch_idx.numel() == batch_size,
                "cache_batch_idx must have shape [batch_size]");
    // Bounds are checked on the host, like the reference (:630-641): an out-of-range row would be
    // an out-of-bounds access on the device.  This is the only synchronising step of this binding.
    if (batch_size > 0) {
      const int64_t lo = cache_batch_idx.min().item<int64_t>();
      const int64_t hi = cache_batch_idx.max().item<int64_t>();
      TORCH_CHECK(lo >= 0 && hi < batch_size_cache, "cache_batch_idx entries must be within cache batch bounds");
    }
  } else {
    TORCH_CHECK(batch_size == batch_size_cache,
                "q and cache batch size must match when cache_batch_idx is not provided");
  }

  at::Tensor k, v;
  const bool has_k = !k_obj.is_none();
  const bool has_v = !v_obj.is_none();
  TORCH_CHECK(has_k == has_v, "k and v must either both be provided or both be None");
  int64_t seqlen_new = 0;
  if (has_k) {
    k = k_obj.cast<at::Tensor>();
    v = v_obj.cast<at::Tensor>();
    TORCH_CHECK(k.is_cuda() && v.is_cuda(), "k and v must be CUDA tensors");
    TORCH_CHECK(k.scalar_type() == torch::kFloat16 && v.scalar_type() == torch::kFloat16,
                "k and v must be float16 tensors");
    TORCH_CHECK(k.dim() == 4 && v.dim() == 4, "k and v must be rank-4 tensors");
    TORCH_CHECK(k.size(0) == batch_size && v.size(0) == batch_size, "k/v batch size must match q");
    TORCH_CHECK(k.size(1) == v.size(1), "k and v seqlen must match");
    TORCH_CHECK(k.size(2) == num_heads_k && v.size(2) == num_heads_k,
                "k/v num_heads must match the cache num_heads");
    TORCH_CHECK(k.size(3) == head_size && v.size(3) == head_size, "k/v head_dim must match q");
    TORCH_CHECK(k.stride(-1) == 1 && v.stride(-1) == 1, "k and v must have contiguous last dimension");
    seqlen_new = k.size(1);
  }
  c10::cuda::CUDAGuard guard(q.device());

  at::Tensor out = torch::empty_like(q, q.options(), at::MemoryFormat::Contiguous);
  at::Tensor lse = torch::empty({batch_size, num_heads, seqlen_q}, q.options().dtype(torch::kFloat32));
  if (batch_size == 0 || seqlen_q == 0) return {out, lse};

  FaKvcacheParams p = {};
  p.q = q.data_ptr(); p.k_cache = k_cache.data_ptr(); p.v_cache = v_cache.data_ptr();
  p.o = out.data_ptr(); p.lse = lse.data_ptr<float>();
  p.q_batch_stride = q.stride(0); p.q_row_stride = q.stride(1); p.q_head_stride = q.stride(2);
  p.kc_batch_stride = k_cache.stride(0); p.kc_row_stride = k_cache.stride(1); p.kc_head_stride = k_cache.stride(2);
  p.vc_batch_stride = v_cache.stride(0); p.vc_row_stride = v_cache.stride(1); p.vc_head_stride = v_cache.stride(2);
  if (has_k && seqlen_new > 0) {
    p.k_new = k.data_ptr(); p.v_new = v.data_ptr();
    p.kn_batch_stride = k.stride(0); p.kn_row_stride = k.stride(1); p.kn_head_stride = k.stride(2);
    p.vn_batch_stride = v.stride(0); p.vn_row_stride = v.stride(1); p.vn_head_stride = v.stride(2);
  }
  p.o_batch_stride = out.stride(0); p.o_row_stride = out.stride(1); p.o_head_stride = out.stride(2);
  p.b = batch_size; p.seqlen_q = seqlen_q; p.seqlen_new = seqlen_new;
  p.h = num_heads; p.h_k = num_heads_k; p.d = head_size;
  p.cache_batch = k_cache.size(0);
  p.seqlen_cache = k_cache.size(1);
  p.softmax_scale = static_cast<float>(softmax_scale);
  p.is_causal = is_causal;
  p.cache_seqlens = cache_seqlens.data_ptr<int>();
  p.cache_batch_idx = has_cache_batch_idx ? cache_batch_idx.data_ptr<int>() : nullptr;
  if (has_block_table) {
    p.block_table = block_table.data_ptr<int>();
    p.block_table_batch_stride = block_table.stride(0);
    p.max_blocks_per_seq = block_table.size(1);
  }
  p.num_splits = static_cast<int32_t>(num_splits);
  const size_t ws = fa_kvcache_workspace_bytes(&p);
  at::Tensor workspace = torch::empty({static_cast<int64_t>(ws)}, q.options().dtype(torch::kUInt8));
  p.workspace = ws ? workspace.data_ptr() : nullptr;
  p.workspace_bytes = ws;
  check_rc(fa_kvcache(&p, current_stream()), "fa_kvcache");
  return {out, lse};
}

// ---- stand-alone LSE merge (no counterpart binding in the reference; used after the NCCL exchange
// of a sequence-sharded forward) ----
std::vector<at::Tensor> combine(at::Tensor o_accum, at::Tensor lse_accum, int64_t b, int64_t seqlen_q,
                                int64_t h) {
  TORCH_CHECK(o_accum.is_cuda() && lse_accum.is_cuda(), "o_accum and lse_accum must be CUDA tensors");
  TORCH_CHECK(o_accum.scalar_type() == torch::kFloat32 && lse_accum.scalar_type() == torch::kFloat32,
              "o_accum and lse_accum must be float32 tensors");
  TORCH_CHECK(o_accum.is_contiguous() && lse_accum.is_contiguous(), "o_accum and lse_accum must be contiguous");
  TORCH_CHECK(o_accum.dim() == 3 && lse_accum.dim() == 2, "o_accum must be (splits, rows, d), lse_accum (splits, rows)");
  const int64_t splits = o_accum.size(0), rows = o_accum.size(1), d = o_accum.size(2);
  TORCH_CHECK(lse_accum.size(0) == splits && lse_accum.size(1) == rows, "lse_accum shape mismatch");
  TORCH_CHECK(rows == b * h * seqlen_q, "rows must equal b * h * seqlen_q");
  check_supported_head_dim(d);
  c10::cuda::CUDAGuard guard(o_accum.device());
  at::Tensor out = torch::empty({b, seqlen_q, h, d}, o_accum.options().dtype(torch::kFloat16));
  at::Tensor lse = torch::empty({b, h, seqlen_q}, o_accum.options());
  if (rows == 0) return {out, lse};
  FaCombineParams p = {};
  p.o_accum = o_accum.data_ptr<float>();
  p.lse_accum = lse_accum.data_ptr<float>();
  p.o = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.o_batch_stride = out.stride(0); p.o_row_stride = out.stride(1); p.o_head_stride = out.stride(2);
  p.num_splits = splits; p.b = b; p.h = h; p.seqlen_q = seqlen_q; p.d = d;
  check_rc(fa_combine(&p, current_stream()), "fa_combine");
  return {out, lse};
}

// ---- merge of per-rank partials read in place (o_parts[r] may be peer-mapped memory of another GPU) ----
std::vector<at::Tensor> combine_gather(std::vector<at::Tensor> o_parts, std::vector<at::Tensor> lse_parts,
                                       int64_t row_begin, int64_t rows) {
  TORCH_CHECK(!o_parts.empty() && o_parts.size() == lse_parts.size(), "o_parts and lse_parts must have the same non-zero length");
  TORCH_CHECK(o_parts.size() <= FA_MAX_GATHER_PARTS, "at most ", FA_MAX_GATHER_PARTS, " parts");
  const at::Tensor& o0 = o_parts[0];
  TORCH_CHECK(o0.dim() == 4, "partial O must be (b, seqlen_q, h, d)");
  const int64_t b = o0.size(0), s = o0.size(1), h = o0.size(2), d = o0.size(3);
  check_supported_head_dim(d);
  FaCombineGatherParams p = {};
  for (size_t i = 0; i < o_parts.size(); ++i) {
    TORCH_CHECK(o_parts[i].is_cuda() && o_parts[i].scalar_type() == at::kHalf && o_parts[i].is_contiguous() &&
                    o_parts[i].sizes() == o0.sizes(),
                "partial O tensors must be contiguous float16 CUDA tensors of one shape");
    TORCH_CHECK(lse_parts[i].is_cuda() && lse_parts[i].scalar_type() == at::kFloat && lse_parts[i].is_contiguous() &&
                    lse_parts[i].dim() == 3 && lse_parts[i].size(0) == b && lse_parts[i].size(1) == h && lse_parts[i].size(2) == s,
                "partial LSE tensors must be contiguous float32 (b, h, seqlen_q) CUDA tensors");
    p.o_part[i] = o_parts[i].data_ptr();
    p.lse_part[i] = lse_parts[i].data_ptr<float>();
  }
  TORCH_CHECK(row_begin >= 0 && rows >= 0 && row_begin + rows <= s, "row range out of bounds");
  // outputs live on the CURRENT device (the partial tensors may be views of peer memory)
  auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
  at::Tensor out = torch::empty({b, rows, h, d}, opts.dtype(torch::kFloat16));
  at::Tensor lse = torch::empty({b, h, rows}, opts.dtype(torch::kFloat32));
  p.o = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.num_parts = static_cast<int32_t>(o_parts.size());
  p.b = b; p.h = h; p.seqlen_q = s; p.d = d;
  p.row_begin = row_begin; p.rows = rows;
  check_rc(fa_combine_gather(&p, current_stream()), "fa_combine_gather");
  return {out, lse};
}

// ---- sum of per-rank partial dQ read in place (parts[r] may be peer-mapped memory of another GPU) ----
// first_rows (optional): per part, the first query row that holds anything (rows below are not read).
at::Tensor sum_gather(std::vector<at::Tensor> parts, int64_t row_begin, int64_t rows,
                      c10::optional<std::vector<int64_t>> first_rows) {
  TORCH_CHECK(!parts.empty() && parts.size() <= FA_MAX_GATHER_PARTS, "between 1 and ", FA_MAX_GATHER_PARTS, " parts");
  const at::Tensor& p0 = parts[0];
  TORCH_CHECK(p0.dim() == 4, "partial dQ must be (b, seqlen_q, h, d)");
  const int64_t b = p0.size(0), s = p0.size(1), h = p0.size(2), d = p0.size(3);
  check_supported_head_dim(d);
  FaSumGatherParams p = {};
  for (size_t i = 0; i < parts.size(); ++i) {
    TORCH_CHECK(parts[i].is_cuda() && parts[i].scalar_type() == at::kHalf && parts[i].is_contiguous() &&
                    parts[i].sizes() == p0.sizes(),
                "partial dQ tensors must be contiguous float16 CUDA tensors of one shape");
    p.part[i] = parts[i].data_ptr();
  }
  if (first_rows.has_value()) {
    TORCH_CHECK(first_rows->size() == parts.size(), "first_rows must have one entry per part");
    for (size_t i = 0; i < parts.size(); ++i) p.part_first_row[i] = static_cast<int32_t>((*first_rows)[i]);
  }
  TORCH_CHECK(row_begin >= 0 && rows >= 0 && row_begin + rows <= s, "row range out of bounds");
  auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
  at::Tensor out = torch::empty({b, rows, h, d}, opts.dtype(torch::kFloat16));
  p.out = out.data_ptr();
  p.num_parts = static_cast<int32_t>(parts.size());
  p.b = b; p.h = h; p.seqlen_q = s; p.d = d;
  p.row_begin = row_begin; p.rows = rows;
  if (b > 0 && rows > 0) check_rc(fa_sum_gather(&p, current_stream()), "fa_sum_gather");
  return out;
}

int64_t device_status(bool reset) { return fa_device_status(reset ? 1 : 0); }

// Which backward path bwd / varlen_bwd use: false (default) = the dQ kernel + the dK/dV kernel, bitwise
// reproducible; true = the single kernel with five products whose dQ accumulation order depends on scheduling
// (FA_BWD_SINGLE_KERNEL).
void set_single_kernel_backward(bool on) { g_bwd_flags = on ? FA_BWD_SINGLE_KERNEL : 0; }
bool get_single_kernel_backward() { return (g_bwd_flags & FA_BWD_SINGLE_KERNEL) != 0; }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("fwd", &mha_fwd, "Forward pass", py::arg("q"), py::arg("k"), py::arg("v"), py::arg("softmax_scale"),
        py::arg("is_causal"), py::arg("out") = py::none(), py::arg("lse") = py::none(),
        py::arg("causal_shift") = py::none());
  m.def("bwd", &mha_bwd, "Backward pass", py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("l"),
        py::arg("dout"), py::arg("softmax_scale"), py::arg("is_causal"), py::arg("dq") = py::none(),
        py::arg("dk") = py::none(), py::arg("dv") = py::none(), py::arg("causal_shift") = py::none());
  m.def("varlen_fwd", &mha_varlen_fwd, "Varlen forward pass");
  m.def("varlen_bwd", &mha_varlen_bwd, "Varlen backward pass", py::arg("q"), py::arg("k"), py::arg("v"),
        py::arg("out"), py::arg("l"), py::arg("dout"), py::arg("cu_seqlens_q"), py::arg("cu_seqlens_k"),
        py::arg("max_seqlen_q"), py::arg("max_seqlen_k"), py::arg("softmax_scale"), py::arg("is_causal"),
        py::arg("dq") = py::none(), py::arg("dk") = py::none(), py::arg("dv") = py::none());
  m.def("fwd_kvcache", &mha_fwd_kvcache, "KV-cache forward pass");
  m.def("combine", &combine, "Merge split partials (O fp32, LSE) with log-sum-exp weights");
  m.def("combine_gather", &combine_gather, "Merge per-rank partial (O fp16, LSE) read in place, peer memory allowed");
  m.def("sum_gather", &sum_gather, "Sum per-rank partial dQ (fp16) read in place, peer memory allowed", py::arg("parts"),
        py::arg("row_begin"), py::arg("rows"), py::arg("first_rows") = py::none());
  m.def("device_status", &device_status, "Synchronise and read the device status word");
  m.def("set_single_kernel_backward", &set_single_kernel_backward,
        "Select the single-kernel backward (true) or the bitwise reproducible two-kernel backward (false, default)");
  m.def("get_single_kernel_backward", &get_single_kernel_backward, "Which backward path is selected");
}
