"""Operator API of the B200 FlashAttention: a drop-in for ``flash_attention_interface.py`` of
Cy-47/flash-attention-turing.

Same seven public functions, argument order, defaults, return types, exception types, messages and
check order as the reference (``flash_attention_interface.py:448-614`` and ``:779-922``), and the
same six ``torch.autograd.Function`` names (``:172-445``).  Everything below the Python layer is
different: the calls go to ``libfa_b200.so`` (hand-written sm_100a kernels) through a thin torch
binding, and there is no CPU or pure-PyTorch execution path -- the reference's own torch fallback
for the KV-cache (``:890-907``) is deliberately not reproduced.

Differences that are visible only as speed:
* packed inputs (``qkv`` / ``kv``) are passed to the kernels as strided views; the reference makes
  contiguous copies of q, k and v first (``:208-212``, ``:244-247``);
* ``flash_attn_with_kvcache`` always runs the native kernels, for every ``num_splits``.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import _ext


# The reference reads cache_seqlens back to the host to check the cache capacity on every call
# (``int(cache_seqlens.max().item())``, its :855) -- a device synchronisation per decode step.  The check
# is part of the reference's error contract, so it stays on by default.  A serving loop that guarantees
# capacity itself can set this to False: the kernels then clamp every length to the capacity on the device
# (never reading or writing out of bounds) and report a clamp through ``device_status()`` bit 1.
HOST_CAPACITY_CHECK = True


def _gpu():
    """The torch binding (loaded on first use so that argument validation works without a GPU)."""
    return _ext.load()


def maybe_contiguous(x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Only the innermost stride has to be 1 (reference ``:9-10``); outer strides are free."""
    if x is not None and x.stride(-1) != 1:
        return x.contiguous()
    return x


def _default_scale(q: torch.Tensor, softmax_scale: Optional[float]) -> float:
    return q.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale


# --------------------------------------------------------------------------------------------
# thin wrappers around the five bindings (reference :13-169)
# --------------------------------------------------------------------------------------------
def _flash_attn_forward(q, k, v, softmax_scale: float, causal: bool):
    q, k, v = (maybe_contiguous(t) for t in (q, k, v))
    out, lse = _gpu().fwd(q, k, v, softmax_scale, causal)
    return out, lse


def _flash_attn_backward(dout, q, k, v, out, lse, softmax_scale: float, causal: bool, grads=()):
    """``grads``: optional (dq, dk, dv) destinations, e.g. views into one packed gradient tensor; the kernels
    write through their strides, so the packed variants need no concatenation afterwards."""
    dout, q, k, v, out, lse = (maybe_contiguous(t) for t in (dout, q, k, v, out, lse))
    dq, dk, dv = _gpu().bwd(q, k, v, out, lse, dout, softmax_scale, causal, *grads)
    return dq, dk, dv


def _flash_attn_varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                               softmax_scale: float, causal: bool):
    q, k, v = (maybe_contiguous(t) for t in (q, k, v))
    out, lse = _gpu().varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                 softmax_scale, causal)
    return out, lse


def _flash_attn_varlen_backward(dout, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int,
                                max_seqlen_k: int, softmax_scale: float, causal: bool, grads=()):
    dout, q, k, v, out, lse = (maybe_contiguous(t) for t in (dout, q, k, v, out, lse))
    dq, dk, dv = _gpu().varlen_bwd(q, k, v, out, lse, dout, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                   max_seqlen_k, softmax_scale, causal, *grads)
    return dq, dk, dv


def _flash_attn_kvcache_forward(q, k_cache, v_cache, k, v, cache_seqlens, cache_batch_idx, block_table,
                                softmax_scale: float, causal: bool, num_splits: int):
    q, k_cache, v_cache, k, v, cache_seqlens, cache_batch_idx, block_table = (
        maybe_contiguous(t) for t in (q, k_cache, v_cache, k, v, cache_seqlens, cache_batch_idx, block_table)
    )
    # 20-argument binding of the reference (flash_api.cpp:508-528); unsupported features are None.
    out, lse = _gpu().fwd_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, None, None, cache_batch_idx,
                                  None, block_table, None, None, softmax_scale, causal, -1, -1, 0.0, True,
                                  num_splits)
    return out, lse


# --------------------------------------------------------------------------------------------
# autograd glue (reference :172-445)
# --------------------------------------------------------------------------------------------
def _save_dense(ctx, needs_grad, q, k, v, out, lse, softmax_scale, causal):
    if needs_grad:
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal


def _dense_backward(ctx, dout, grads=()):
    q, k, v, out, lse = ctx.saved_tensors
    return _flash_attn_backward(dout, q, k, v, out, lse, ctx.softmax_scale, ctx.causal, grads)


def _packed_like(parts, dim):
    """One packed gradient tensor for ``parts`` (same-shape q/k/v views) stacked along ``dim``, and its
    unbound views: the layout the reference builds by concatenation (:226-231, :262-264)."""
    shape = list(parts[0].shape)
    shape.insert(dim, len(parts))
    packed = torch.empty(shape, dtype=parts[0].dtype, device=parts[0].device)
    return packed, packed.unbind(dim=dim)


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, is_grad_enabled):
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_forward(q, k, v, softmax_scale, causal)
        _save_dense(ctx, is_grad_enabled and any(t.requires_grad for t in (q, k, v)),
                    q, k, v, out, lse, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        dq, dk, dv = _dense_backward(ctx, dout)
        return dq, dk, dv, None, None, None


class FlashAttnQKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, softmax_scale, causal, is_grad_enabled):
        q, k, v = qkv.unbind(dim=2)  # strided views of (b, s, 3, h, d); no copies
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_forward(q, k, v, softmax_scale, causal)
        _save_dense(ctx, is_grad_enabled and qkv.requires_grad, q, k, v, out, lse, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v = ctx.saved_tensors[:3]
        dqkv, views = _packed_like((q, k, v), 2)
        _dense_backward(ctx, dout, views)
        return dqkv, None, None, None


class FlashAttnKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, softmax_scale, causal, is_grad_enabled):
        k, v = kv.unbind(dim=2)
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_forward(q, k, v, softmax_scale, causal)
        _save_dense(ctx, is_grad_enabled and any(t.requires_grad for t in (q, kv)),
                    q, k, v, out, lse, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v = ctx.saved_tensors[:3]
        dkv, (dk, dv) = _packed_like((k, v), 2)
        dq, _, _ = _dense_backward(ctx, dout, (torch.empty_like(q), dk, dv))
        return dq, dkv, None, None, None


def _save_varlen(ctx, needs_grad, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, softmax_scale, causal):
    if needs_grad:
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.max_seqlen_q = max_q
        ctx.max_seqlen_k = max_k
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal


def _varlen_backward(ctx, dout, grads=()):
    q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
    return _flash_attn_varlen_backward(dout, q, k, v, out, lse, cu_q, cu_k, ctx.max_seqlen_q,
                                       ctx.max_seqlen_k, ctx.softmax_scale, ctx.causal, grads)


class FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                is_grad_enabled):
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                              softmax_scale, causal)
        _save_varlen(ctx, is_grad_enabled and any(t.requires_grad for t in (q, k, v)), q, k, v, out, lse,
                     cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        dq, dk, dv = _varlen_backward(ctx, dout)
        return dq, dk, dv, None, None, None, None, None, None, None


class FlashAttnVarlenQKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, softmax_scale, causal, is_grad_enabled):
        q, k, v = qkv.unbind(dim=1)  # (total, 3, h, d) -> three strided (total, h, d) views
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_varlen_forward(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                              softmax_scale, causal)
        _save_varlen(ctx, is_grad_enabled and qkv.requires_grad, q, k, v, out, lse, cu_seqlens, cu_seqlens,
                     max_seqlen, max_seqlen, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v = ctx.saved_tensors[:3]
        dqkv, views = _packed_like((q, k, v), 1)
        _varlen_backward(ctx, dout, views)
        return dqkv, None, None, None, None, None


class FlashAttnVarlenKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                is_grad_enabled):
        k, v = kv.unbind(dim=1)
        softmax_scale = _default_scale(q, softmax_scale)
        out, lse = _flash_attn_varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                              softmax_scale, causal)
        _save_varlen(ctx, is_grad_enabled and any(t.requires_grad for t in (q, kv)), q, k, v, out, lse,
                     cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v = ctx.saved_tensors[:3]
        dkv, (dk, dv) = _packed_like((k, v), 1)
        dq, _, _ = _varlen_backward(ctx, dout, (torch.empty_like(q), dk, dv))
        return dq, dkv, None, None, None, None, None, None, None


# --------------------------------------------------------------------------------------------
# public functions (reference :448-614)
# --------------------------------------------------------------------------------------------
def flash_attn_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: Optional[float] = None,
                    causal: bool = False) -> torch.Tensor:
    """q (batch, seqlen_q, nheads, d); k, v (batch, seqlen_k, nheads_k, d) -> out like q.
    nheads must be a multiple of nheads_k (GQA/MQA); d is 64 or 128; fp16.  ``causal`` masks with
    bottom-right alignment.  ``softmax_scale`` defaults to d ** -0.5."""
    return FlashAttnFunc.apply(q, k, v, softmax_scale, causal, torch.is_grad_enabled())


def flash_attn_qkvpacked_func(qkv: torch.Tensor, softmax_scale: Optional[float] = None,
                              causal: bool = False) -> torch.Tensor:
    """qkv (batch, seqlen, 3, nheads, d) -> out (batch, seqlen, nheads, d)."""
    return FlashAttnQKVPackedFunc.apply(qkv, softmax_scale, causal, torch.is_grad_enabled())


def flash_attn_kvpacked_func(q: torch.Tensor, kv: torch.Tensor, softmax_scale: Optional[float] = None,
                             causal: bool = False) -> torch.Tensor:
    """q (batch, seqlen_q, nheads, d); kv (batch, seqlen_k, 2, nheads_k, d) -> out like q."""
    return FlashAttnKVPackedFunc.apply(q, kv, softmax_scale, causal, torch.is_grad_enabled())


def flash_attn_varlen_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                           cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                           softmax_scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
    """Packed sequences: q (total_q, nheads, d); k, v (total_k, nheads_k, d); cu_seqlens_* int32
    (batch + 1,) cumulative offsets; max_seqlen_* the longest sequence.  -> out (total_q, nheads, d)."""
    return FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                     softmax_scale, causal, torch.is_grad_enabled())


def flash_attn_varlen_qkvpacked_func(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                                     softmax_scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
    """qkv (total, 3, nheads, d) with one cu_seqlens for q and k -> out (total, nheads, d)."""
    return FlashAttnVarlenQKVPackedFunc.apply(qkv, cu_seqlens, max_seqlen, softmax_scale, causal,
                                              torch.is_grad_enabled())


def flash_attn_varlen_kvpacked_func(q: torch.Tensor, kv: torch.Tensor, cu_seqlens_q: torch.Tensor,
                                    cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                                    softmax_scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
    """q (total_q, nheads, d); kv (total_k, 2, nheads_k, d) -> out (total_q, nheads, d)."""
    return FlashAttnVarlenKVPackedFunc.apply(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                             softmax_scale, causal, torch.is_grad_enabled())


# --------------------------------------------------------------------------------------------
# KV-cache inference (reference :617-639, :779-922)
# --------------------------------------------------------------------------------------------
def _validate_unsupported_kvcache_args(rotary_cos, rotary_sin, cache_leftpad, window_size, softcap,
                                       alibi_slopes) -> None:
    # Messages kept verbatim: callers and the reference's tests match on them.
    if rotary_cos is not None or rotary_sin is not None:
        raise NotImplementedError("Turing KV-cache does not support rotary embeddings yet")
    if cache_leftpad is not None:
        raise NotImplementedError("Turing KV-cache does not support cache_leftpad yet")
    if window_size != (-1, -1):
        raise NotImplementedError("Turing KV-cache does not support local window attention yet")
    if softcap != 0.0:
        raise NotImplementedError("Turing KV-cache does not support softcap yet")
    if alibi_slopes is not None:
        raise NotImplementedError("Turing KV-cache does not support ALiBi yet")


def _validate_supported_head_dim(head_dim: int) -> None:
    if head_dim not in (64, 128):
        raise ValueError("Turing FlashAttention supports head_dim 64 or 128")


def _require_int32_tensor(x, name: str) -> None:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if x.dtype != torch.int32:
        raise TypeError(f"{name} must be a torch.int32 tensor")


def flash_attn_with_kvcache(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    k: Optional[torch.Tensor] = None,
    v: Optional[torch.Tensor] = None,
    rotary_cos: Optional[torch.Tensor] = None,
    rotary_sin: Optional[torch.Tensor] = None,
    cache_seqlens: Optional[Union[torch.Tensor, int]] = None,
    cache_batch_idx: Optional[torch.Tensor] = None,
    cache_leftpad: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[int, int] = (-1, -1),
    softcap: float = 0.0,
    rotary_interleaved: bool = True,
    alibi_slopes: Optional[torch.Tensor] = None,
    num_splits: int = 0,
    return_softmax_lse: bool = False,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Inference step against a KV cache; signature of upstream FlashAttention.

    Appends ``k``/``v`` (batch, seqlen_new, nheads_k, d) in place at ``cache_seqlens`` and attends
    ``q`` (batch, seqlen_q, nheads, d) against the first ``cache_seqlens + seqlen_new`` tokens.
    Cache layouts: contiguous (batch_cache, seqlen_cache, nheads_k, d), optionally indexed through
    ``cache_batch_idx``; or paged (num_pages, page_size, nheads_k, d) with ``block_table`` (batch,
    max_pages) and page_size % 256 == 0.  ``num_splits`` 0 picks a split count from the shape.
    Rotary, ALiBi, local windows, softcap and cache_leftpad raise NotImplementedError.
    Returns ``out`` or ``(out, softmax_lse)``.
    """
    _validate_unsupported_kvcache_args(rotary_cos, rotary_sin, cache_leftpad, window_size, softcap, alibi_slopes)
    if (k is None) != (v is None):
        raise ValueError("k and v must either both be provided or both be None")
    _validate_supported_head_dim(q.shape[-1])
    batch = q.shape[0]
    capacity = k_cache.shape[1] if block_table is None else block_table.shape[1] * k_cache.shape[1]

    if cache_seqlens is None:
        if k is not None:
            raise ValueError("cache_seqlens is required when appending k and v")
        cache_seqlens = capacity
    if isinstance(cache_seqlens, int):  # bool included, as in the reference (its :818)
        cache_seqlens = torch.full((batch,), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    elif not isinstance(cache_seqlens, torch.Tensor):
        raise TypeError("cache_seqlens must be an int or a torch.Tensor")
    elif cache_seqlens.dtype != torch.int32:
        raise TypeError("cache_seqlens must be a torch.int32 tensor")
    if cache_seqlens.dim() != 1 or cache_seqlens.numel() != batch:
        raise ValueError("cache_seqlens must have shape [batch_size]")

    if block_table is not None:
        _require_int32_tensor(block_table, "block_table")
        if block_table.dim() != 2 or block_table.shape[0] != batch:
            raise ValueError("block_table must have shape [batch_size, max_num_blocks_per_seq]")
        if cache_batch_idx is not None:
            raise NotImplementedError("Paged KV cache does not support cache_batch_idx")
        if k_cache.shape[1] % 256 != 0:
            raise ValueError("Paged KV cache block size must be divisible by 256")
    if cache_batch_idx is not None:
        _require_int32_tensor(cache_batch_idx, "cache_batch_idx")
        if cache_batch_idx.dim() != 1 or cache_batch_idx.numel() != batch:
            raise ValueError("cache_batch_idx must have shape [batch_size]")
    if num_splits < 0:
        raise ValueError("num_splits must be non-negative")

    seqlen_new = 0
    if k is not None:
        if k.shape[0] != batch or v.shape[0] != batch:
            raise ValueError("k and v batch size must match q")
        if k.shape[1] != v.shape[1]:
            raise ValueError("k and v sequence length must match")
        seqlen_new = k.shape[1]
    # Capacity is checked before the device/dtype checks, on whatever device the lengths live
    # (the reference does the same, :855-858, and its tests rely on that order with CPU tensors).
    if HOST_CAPACITY_CHECK or not cache_seqlens.is_cuda:
        used = int(cache_seqlens.max().item()) if cache_seqlens.numel() > 0 else 0
        if used + seqlen_new > capacity:
            raise ValueError("cache capacity is insufficient for the requested append length")

    if not (q.is_cuda and k_cache.is_cuda and v_cache.is_cuda):
        raise RuntimeError("q, k_cache, v_cache must be CUDA tensors")
    if not (q.dtype == k_cache.dtype == v_cache.dtype == torch.float16):
        raise RuntimeError("q, k_cache, v_cache must be float16 tensors")
    if k is not None:
        if not (k.is_cuda and v.is_cuda):
            raise RuntimeError("k and v must be CUDA tensors")
        if k.dtype != torch.float16 or v.dtype != torch.float16:
            raise RuntimeError("k and v must be float16 tensors")

    out, lse = _flash_attn_kvcache_forward(q, k_cache, v_cache, k, v, cache_seqlens, cache_batch_idx,
                                           block_table, _default_scale(q, softmax_scale), causal, num_splits)
    return (out, lse) if return_softmax_lse else out
