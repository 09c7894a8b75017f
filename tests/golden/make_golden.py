"""Generates the golden fixtures in this directory by running the REFERENCE's own Python functions.

Run where the reference checkout is present, giving its root as the argument or in
$FA_REFERENCE_ROOT:

    python tests/golden/make_golden.py <reference root>

The reference's ``flash_attention_interface.py`` imports its CUDA extension at module import time;
a stub module stands in for it (none of the functions used here touch the extension):

* ``_attention_forward_ref``            (flash_attention_interface.py:731-776)  forward + LSE, split-KV
* ``_copy_kv_to_contiguous_cache``      (:642-662)   in-place append, contiguous cache
* ``_copy_kv_to_paged_cache``           (:665-685)   in-place append, paged cache
* ``_materialize_kv_cache``             (:688-728)   gather of a (paged) cache
* gradients: torch.autograd through ``_attention_forward_ref`` evaluated on fp32 copies of the
  fp16 inputs (the reference ships no explicit backward math; its tests use autograd as well,
  test_flash_attn.py:341-361).

Outputs: one ``.npz`` per case with the fp16 inputs and the fp32 reference outputs.  The fixtures are
small (tens of KB) and committed; this script is committed so that they can be regenerated.
"""
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

REF_ROOT = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA_REFERENCE_ROOT")
OUT_DIR = Path(__file__).resolve().parent


def load_reference():
    if not REF_ROOT or not Path(REF_ROOT, "flash_attention_interface.py").is_file():
        raise SystemExit("give the root of the reference checkout as the argument or in $FA_REFERENCE_ROOT")
    sys.modules.setdefault("flash_attn_turing", types.ModuleType("flash_attn_turing"))
    sys.path.insert(0, REF_ROOT)
    import flash_attention_interface as ref  # noqa: E402

    return ref


def rnd(gen, *shape):
    return torch.randn(*shape, generator=gen).half()


def rnd_int(gen, *shape):
    """Small-integer fp16 values: enough to check copies exactly, and they compress well."""
    return torch.randint(-3, 4, shape, generator=gen).half()


def forward_case(ref, name, seed, b, sq, sk_cap, h, hk, d, lens, causal, splits, with_grads):
    gen = torch.Generator().manual_seed(seed)
    q, k, v = rnd(gen, b, sq, h, d), rnd(gen, b, sk_cap, hk, d), rnd(gen, b, sk_cap, hk, d)
    dout = rnd(gen, b, sq, h, d)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    out, lse = ref._attention_forward_ref(q.float(), k.float(), v.float(), lens_t, scale, causal, splits)
    data = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=dout.numpy(), lens=lens_t.numpy(),
                scale=np.float32(scale), causal=np.int32(causal), splits=np.int32(splits),
                out=out.float().numpy(), lse=lse.numpy())
    if with_grads:
        qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
        o2, _ = ref._attention_forward_ref(qf, kf, vf, lens_t, scale, causal, 1)
        dq, dk, dv = torch.autograd.grad(o2, (qf, kf, vf), dout.float())
        data.update(dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())
    np.savez_compressed(OUT_DIR / f"{name}.npz", **data)
    print("wrote", name)


def cache_case(ref, name, seed, paged):
    gen = torch.Generator().manual_seed(seed)
    b, hk, d, s_new = 3, 1, 64, 2
    lens = torch.tensor([5, 0, 300], dtype=torch.int32)
    rnd = rnd_int
    k_new, v_new = rnd(gen, b, s_new, hk, d), rnd(gen, b, s_new, hk, d)
    if paged:
        page, n_pages, per_seq = 256, 8, 2
        k_cache, v_cache = rnd(gen, n_pages, page, hk, d), rnd(gen, n_pages, page, hk, d)
        table = torch.tensor([[3, 6], [0, 5], [7, 1]], dtype=torch.int32)
        k0, v0 = k_cache.clone(), v_cache.clone()
        ref._copy_kv_to_paged_cache(k_cache, v_cache, k_new, v_new, lens, table)
        k_used, v_used = ref._materialize_kv_cache(k_cache, v_cache, lens + s_new, None, table)
        extra = dict(block_table=table.numpy())
    else:
        cap, rows = 320, 5
        k_cache, v_cache = rnd(gen, rows, cap, hk, d), rnd(gen, rows, cap, hk, d)
        idx = torch.tensor([4, 0, 2], dtype=torch.int32)
        k0, v0 = k_cache.clone(), v_cache.clone()
        ref._copy_kv_to_contiguous_cache(k_cache, v_cache, k_new, v_new, lens, idx)
        k_used, v_used = ref._materialize_kv_cache(k_cache, v_cache, lens + s_new, idx, None)
        extra = dict(cache_batch_idx=idx.numpy())
    np.savez_compressed(OUT_DIR / f"{name}.npz", k_cache_before=k0.numpy(), v_cache_before=v0.numpy(),
                        k_new=k_new.numpy(), v_new=v_new.numpy(), lens=lens.numpy(),
                        k_cache_after=k_cache.numpy(), v_cache_after=v_cache.numpy(),
                        k_used=k_used.numpy(), v_used=v_used.numpy(), **extra)
    print("wrote", name)


def main():
    ref = load_reference()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    #            name                   seed b  sq  cap  h hk  d   lens        causal splits grads
    forward_case(ref, "fwd_d64_noncausal", 11, 2, 20, 40, 2, 1, 64, [40, 17], False, 1, True)
    forward_case(ref, "fwd_d64_causal", 12, 2, 20, 40, 2, 2, 64, [40, 17], True, 1, True)
    forward_case(ref, "fwd_d128_causal_gqa", 13, 1, 17, 70, 4, 1, 128, [70], True, 1, True)
    forward_case(ref, "fwd_d128_sq_gt_sk", 14, 1, 30, 12, 2, 2, 128, [12], True, 1, True)
    forward_case(ref, "fwd_d64_split3", 15, 2, 3, 150, 2, 1, 64, [150, 71], True, 3, False)
    forward_case(ref, "fwd_d128_decode_split4", 16, 3, 1, 140, 4, 2, 128, [140, 1, 65], True, 4, False)
    cache_case(ref, "cache_contiguous", 21, paged=False)
    cache_case(ref, "cache_paged", 22, paged=True)


if __name__ == "__main__":
    main()
