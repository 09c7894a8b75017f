"""Host-side behaviour of the operator API that needs no GPU: the argument checks of
flash_attn_with_kvcache (exception type, message and ORDER, which the reference's tests pin with CPU
tensors, test_flash_attn.py:1967-2093 of Cy-47/flash-attention-turing), the public surface, and the
absence of any CPU execution path."""
import inspect

import pytest
import torch

import flash_attention_turing_b200 as fa
from flash_attention_turing_b200 import flash_attention_interface as iface
from flash_attention_turing_b200 import flash_attn_with_kvcache


def _qkv(b=1, sq=2, h=4, hk=2, d=64, cap=8, rows=None):
    rows = b if rows is None else rows
    return torch.randn(b, sq, h, d), torch.randn(rows, cap, hk, d), torch.randn(rows, cap, hk, d)


def test_public_surface_matches_reference():
    names = ["flash_attn_func", "flash_attn_kvpacked_func", "flash_attn_qkvpacked_func", "flash_attn_varlen_func",
             "flash_attn_varlen_kvpacked_func", "flash_attn_varlen_qkvpacked_func", "flash_attn_with_kvcache"]
    for n in names:
        assert callable(getattr(fa, n)) and callable(getattr(iface, n))
    for n in ["FlashAttnFunc", "FlashAttnQKVPackedFunc", "FlashAttnKVPackedFunc", "FlashAttnVarlenFunc",
              "FlashAttnVarlenQKVPackedFunc", "FlashAttnVarlenKVPackedFunc"]:
        assert issubclass(getattr(iface, n), torch.autograd.Function)
    sig = inspect.signature(flash_attn_with_kvcache)
    assert list(sig.parameters) == [
        "q", "k_cache", "v_cache", "k", "v", "rotary_cos", "rotary_sin", "cache_seqlens", "cache_batch_idx",
        "cache_leftpad", "block_table", "softmax_scale", "causal", "window_size", "softcap", "rotary_interleaved",
        "alibi_slopes", "num_splits", "return_softmax_lse"]
    assert sig.parameters["num_splits"].default == 0 and sig.parameters["window_size"].default == (-1, -1)
    assert list(inspect.signature(fa.flash_attn_func).parameters) == ["q", "k", "v", "softmax_scale", "causal"]
    assert list(inspect.signature(fa.flash_attn_varlen_func).parameters) == [
        "q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q", "max_seqlen_k", "softmax_scale", "causal"]


def test_append_needs_cache_seqlens():
    q, kc, vc = _qkv()
    with pytest.raises(ValueError, match="cache_seqlens is required when appending"):
        flash_attn_with_kvcache(q, kc, vc, k=torch.randn(1, 1, 2, 64), v=torch.randn(1, 1, 2, 64))


def test_k_and_v_go_together():
    q, kc, vc = _qkv()
    with pytest.raises(ValueError, match="k and v must either both be provided"):
        flash_attn_with_kvcache(q, kc, vc, k=torch.randn(1, 2, 2, 64), cache_seqlens=torch.tensor([4], dtype=torch.int32))


def test_cache_seqlens_dtype_and_shape():
    q, kc, vc = _qkv()
    with pytest.raises(TypeError, match="cache_seqlens must be a torch.int32 tensor"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor([4], dtype=torch.int64))
    with pytest.raises(TypeError, match="cache_seqlens must be an int or a torch.Tensor"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=4.0)
    q2, kc2, vc2 = _qkv(b=2)
    with pytest.raises(ValueError, match=r"cache_seqlens must have shape \[batch_size\]"):
        flash_attn_with_kvcache(q2, kc2, vc2, cache_seqlens=torch.tensor([4], dtype=torch.int32))


def test_cpu_tensors_are_rejected_not_computed():
    # No CPU path exists: valid arguments on CPU tensors end in the reference's RuntimeError.
    q, kc, vc = _qkv()
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor([4], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=4)  # int form


def test_head_dim_check():
    q, kc, vc = _qkv(d=96)
    with pytest.raises(ValueError, match="head_dim 64 or 128"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor([4], dtype=torch.int32))


def test_cache_batch_idx_checks():
    q, kc, vc = _qkv(rows=2)
    lens = torch.tensor([4], dtype=torch.int32)
    with pytest.raises(TypeError, match="cache_batch_idx must be a torch.int32 tensor"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, cache_batch_idx=torch.tensor([1], dtype=torch.int64))
    q2, kc2, vc2 = _qkv(b=2, rows=3)
    with pytest.raises(ValueError, match=r"cache_batch_idx must have shape \[batch_size\]"):
        flash_attn_with_kvcache(q2, kc2, vc2, cache_seqlens=torch.tensor([4, 5], dtype=torch.int32),
                                cache_batch_idx=torch.tensor([1], dtype=torch.int32))


def test_capacity_is_checked_before_device():
    q, kc, vc = _qkv(cap=5)
    with pytest.raises(ValueError, match="cache capacity is insufficient"):
        flash_attn_with_kvcache(q, kc, vc, k=torch.randn(1, 2, 2, 64), v=torch.randn(1, 2, 2, 64),
                                cache_seqlens=torch.tensor([4], dtype=torch.int32))


def test_block_table_checks():
    q = torch.randn(2, 1, 4, 64)
    kc, vc = torch.randn(4, 256, 2, 64), torch.randn(4, 256, 2, 64)
    lens = torch.tensor([4, 5], dtype=torch.int32)
    with pytest.raises(TypeError, match="block_table must be a torch.int32 tensor"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, block_table=torch.zeros(2, 2, dtype=torch.int64))
    with pytest.raises(ValueError, match=r"block_table must have shape \[batch_size, max_num_blocks_per_seq\]"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, block_table=torch.zeros(1, 2, dtype=torch.int32))
    with pytest.raises(NotImplementedError, match="Paged KV cache does not support cache_batch_idx"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens, block_table=torch.zeros(2, 2, dtype=torch.int32),
                                cache_batch_idx=torch.zeros(2, dtype=torch.int32))
    kc3, vc3 = torch.randn(4, 128, 2, 64), torch.randn(4, 128, 2, 64)
    with pytest.raises(ValueError, match="block size must be divisible by 256"):
        flash_attn_with_kvcache(q, kc3, vc3, cache_seqlens=lens, block_table=torch.zeros(2, 2, dtype=torch.int32))


@pytest.mark.parametrize("kwargs,msg", [
    (dict(rotary_cos=torch.zeros(1)), "rotary embeddings"),
    (dict(cache_leftpad=torch.zeros(1)), "cache_leftpad"),
    (dict(window_size=(4, 0)), "local window attention"),
    (dict(softcap=1.0), "softcap"),
    (dict(alibi_slopes=torch.zeros(1)), "ALiBi"),
])
def test_unsupported_features_raise_first(kwargs, msg):
    q, kc, vc = _qkv(d=96)  # the head_dim error must not come first
    with pytest.raises(NotImplementedError, match=msg):
        flash_attn_with_kvcache(q, kc, vc, **kwargs)


def test_negative_num_splits():
    q, kc, vc = _qkv()
    with pytest.raises(ValueError, match="num_splits must be non-negative"):
        flash_attn_with_kvcache(q, kc, vc, cache_seqlens=torch.tensor([4], dtype=torch.int32), num_splits=-1)


def test_dense_ops_reject_cpu_tensors():
    # flash_attn_func on CPU tensors reaches the binding, which refuses them: there is no CPU kernel.
    from flash_attention_turing_b200 import _ext
    if not _ext.EXT_PATH.exists():
        pytest.skip("native extension not built")
    q = torch.randn(1, 4, 2, 64).half()
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fa.flash_attn_func(q, q, q)
