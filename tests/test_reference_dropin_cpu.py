"""Drop-in check against the reference's OWN Python layer, where its checkout is at hand.

The reference's ``flash_attention_interface.py`` does ``import flash_attn_turing as flash_attn_gpu``
(``flash_attention_interface.py:5``).  Here that name is bound to this package's binding module, the
reference's Python file is imported unmodified on top of it, and

* every public function of the reference is compared with ours parameter by parameter (name, kind,
  default), so that a change on either side is caught without a hand-kept list;
* the binding module offers the five functions the reference's Python calls, by name;
* calls with CPU tensors travel through the reference's Python into our binding and are refused
  there (no CPU kernel exists), while the argument errors the reference raises in Python
  (``flash_attention_interface.py:807-867``) come out in the same order from both layers.

The checkout is looked up in ``$FA_REFERENCE_ROOT``, else in a directory ``reference`` beside this
repository; without one the tests are skipped.  No GPU is needed.
"""
import importlib.util
import inspect
import os
import sys
from pathlib import Path

import pytest
import torch

import flash_attention_turing_b200 as fa
from flash_attention_turing_b200 import _ext

REPO = Path(__file__).resolve().parents[1]
REF_ROOT = Path(os.environ.get("FA_REFERENCE_ROOT", REPO.parent / "reference"))
REF_FILE = REF_ROOT / "flash_attention_interface.py"

PUBLIC = ["flash_attn_func", "flash_attn_kvpacked_func", "flash_attn_qkvpacked_func", "flash_attn_varlen_func",
          "flash_attn_varlen_kvpacked_func", "flash_attn_varlen_qkvpacked_func", "flash_attn_with_kvcache"]
FUNCTIONS = ["FlashAttnFunc", "FlashAttnQKVPackedFunc", "FlashAttnKVPackedFunc", "FlashAttnVarlenFunc",
             "FlashAttnVarlenQKVPackedFunc", "FlashAttnVarlenKVPackedFunc"]
BINDINGS = ["fwd", "bwd", "varlen_fwd", "varlen_bwd", "fwd_kvcache"]


@pytest.fixture(scope="module")
def ref():
    if not REF_FILE.is_file():
        pytest.skip("no reference checkout beside the repository")
    if not _ext.EXT_PATH.exists() or not _ext.LIB_PATH.exists():
        pytest.skip("native extension not built")
    saved = sys.modules.get("flash_attn_turing")
    sys.modules["flash_attn_turing"] = _ext.load()
    try:
        spec = importlib.util.spec_from_file_location("_reference_interface", REF_FILE)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        yield module
    finally:
        if saved is None:
            sys.modules.pop("flash_attn_turing", None)
        else:
            sys.modules["flash_attn_turing"] = saved


@pytest.mark.parametrize("name", PUBLIC)
def test_signature_equals_the_reference(ref, name):
    theirs = inspect.signature(getattr(ref, name)).parameters
    ours = inspect.signature(getattr(fa, name)).parameters
    assert list(ours) == list(theirs)
    for key in theirs:
        assert ours[key].kind == theirs[key].kind, key
        assert ours[key].default == theirs[key].default, key


def test_autograd_functions_and_bindings_exist(ref):
    from flash_attention_turing_b200 import flash_attention_interface as iface
    for name in FUNCTIONS:
        assert issubclass(getattr(ref, name), torch.autograd.Function)
        assert issubclass(getattr(iface, name), torch.autograd.Function)
    for name in BINDINGS:
        assert callable(getattr(ref.flash_attn_gpu, name)), name


def test_reference_python_reaches_our_binding_and_is_refused_on_cpu(ref):
    q = torch.randn(1, 4, 2, 64).half()
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ref.flash_attn_func(q, q, q)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    qv = torch.randn(4, 2, 64).half()
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ref.flash_attn_varlen_func(qv, qv, qv, cu, cu, 4, 4)


def test_reference_helpers_bind_every_argument_of_our_bindings(ref):
    """The reference's private helpers call ``bwd``, ``varlen_bwd`` and ``fwd_kvcache`` positionally
    (``flash_attention_interface.py:42-51, 96-109, 131-152``).  With CPU tensors each call must get past
    pybind's argument matching (no ``TypeError``: the reference would answer one from ``fwd_kvcache`` with
    its legacy nine-argument call, ``:153-168``) and be refused by the binding's own device check."""
    q = torch.randn(1, 4, 2, 64).half()
    lse = torch.zeros(1, 2, 4)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ref._flash_attn_backward(q, q, q, q, q, lse, 0.125, True)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ref._flash_attn_varlen_backward(q[0], q[0], q[0], q[0], q[0], lse, cu, cu, 4, 4, 0.125, True)
    cache = torch.randn(1, 8, 2, 64).half()
    lens = torch.tensor([4], dtype=torch.int32)
    idx = torch.zeros(1, dtype=torch.int32)
    for args in [(q, cache, cache, None, None, lens, None, None, 0.125, True, 0),
                 (q, cache, cache, q[:, :1], q[:, :1], lens, idx, None, 0.125, True, 2),
                 (q, torch.randn(2, 256, 2, 64).half(), torch.randn(2, 256, 2, 64).half(), None, None, lens, None,
                  torch.zeros(1, 1, dtype=torch.int32), 0.125, True, 4)]:
        with pytest.raises(RuntimeError, match="must be CUDA tensors"):
            ref._flash_attn_kvcache_forward(*args)


def _kvcache_cases():
    q = torch.randn(1, 2, 4, 64)
    kc, vc = torch.randn(1, 8, 2, 64), torch.randn(1, 8, 2, 64)
    k_new = torch.randn(1, 2, 2, 64)
    lens = torch.tensor([4], dtype=torch.int32)
    yield "append without cache_seqlens", dict(q=q, k_cache=kc, v_cache=vc, k=k_new, v=k_new)
    yield "k without v", dict(q=q, k_cache=kc, v_cache=vc, k=k_new, cache_seqlens=lens)
    yield "cache_seqlens dtype", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens.long())
    yield "cache_seqlens shape", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=torch.zeros(3, dtype=torch.int32))
    yield "rotary", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens, rotary_cos=torch.zeros(8, 16))
    yield "window", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens, window_size=(4, 0))
    yield "softcap", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens, softcap=1.0)
    yield "negative splits", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens, num_splits=-1)
    yield "capacity", dict(q=q, k_cache=kc, v_cache=vc, k=k_new, v=k_new,
                           cache_seqlens=torch.tensor([7], dtype=torch.int32))
    yield "head dim", dict(q=torch.randn(1, 2, 4, 32), k_cache=torch.randn(1, 8, 2, 32),
                           v_cache=torch.randn(1, 8, 2, 32), cache_seqlens=lens)
    yield "valid arguments on CPU tensors", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens)
    yield "valid append on CPU tensors", dict(q=q, k_cache=kc, v_cache=vc, k=k_new, v=k_new, cache_seqlens=lens)
    yield "append shorter than q", dict(q=q, k_cache=kc, v_cache=vc, k=k_new[:, :1], v=k_new[:, :1],
                                        cache_seqlens=lens)
    yield "cache_batch_idx dtype", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens,
                                        cache_batch_idx=torch.zeros(1, dtype=torch.int64))
    yield "cache_batch_idx shape", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens,
                                        cache_batch_idx=torch.zeros(2, dtype=torch.int32))
    yield "alibi", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens, alibi_slopes=torch.zeros(4))
    yield "leftpad", dict(q=q, k_cache=kc, v_cache=vc, cache_seqlens=lens,
                          cache_leftpad=torch.zeros(1, dtype=torch.int32))
    yield "float64 q on CPU", dict(q=q.double(), k_cache=kc, v_cache=vc, cache_seqlens=lens)
    yield "paged with cache_batch_idx", dict(
        q=q, k_cache=torch.randn(2, 256, 2, 64), v_cache=torch.randn(2, 256, 2, 64), cache_seqlens=lens,
        block_table=torch.zeros(1, 1, dtype=torch.int32), cache_batch_idx=torch.zeros(1, dtype=torch.int32))


def _outcome(fn, kwargs):
    try:
        fn(**kwargs)
    except Exception as exc:  # noqa: BLE001  (the type and the text are what is compared)
        return type(exc), str(exc)
    return None, ""


@pytest.mark.parametrize("label,kwargs", list(_kvcache_cases()), ids=[c[0] for c in _kvcache_cases()])
def test_kvcache_argument_errors_equal_the_reference(ref, label, kwargs):
    """Same exception type and text for the same call: the checks run in the reference's order
    (``flash_attention_interface.py:807-867``), so the FIRST failing check decides, and a call whose
    arguments are all valid still ends at the CUDA-tensor check (``:859-866``) on both sides."""
    their_type, their_text = _outcome(ref.flash_attn_with_kvcache, kwargs)
    our_type, our_text = _outcome(fa.flash_attn_with_kvcache, kwargs)
    assert their_type is not None, "the reference accepted a call on CPU tensors"
    assert our_type is their_type, (their_text, our_text)
    assert our_text == their_text
