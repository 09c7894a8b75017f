"""Pins the CPU oracle against fixtures generated from the reference's own Python functions
(tests/golden/make_golden.py).  No GPU needed."""
import pytest
import torch

from helpers import load_golden, t
from oracle import attention_oracle as orc

FWD_CASES = ["fwd_d64_noncausal", "fwd_d64_causal", "fwd_d128_causal_gqa", "fwd_d128_sq_gt_sk"]
SPLIT_CASES = ["fwd_d64_split3", "fwd_d128_decode_split4"]


def _normalise_lse(lse):
    # the reference's torch math yields -inf for rows without a visible key; its tests map that to 0
    return torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))


@pytest.mark.parametrize("name", FWD_CASES + SPLIT_CASES)
def test_forward_matches_reference_math(name):
    g = load_golden(name)
    q, k, v = t(g["q"]), t(g["k"]), t(g["v"])
    out, lse = orc.attention_forward(q, k, v, float(g["scale"]), bool(g["causal"]), seqlens_k=g["lens"].tolist())
    ref_out = t(g["out"])
    ref_out = torch.where(torch.isfinite(ref_out), ref_out, torch.zeros_like(ref_out))
    torch.testing.assert_close(out, ref_out, atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(lse, _normalise_lse(t(g["lse"])), atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("name", FWD_CASES)
def test_backward_matches_autograd_through_reference_math(name):
    g = load_golden(name)
    q, k, v, dout = t(g["q"]), t(g["k"]), t(g["v"]), t(g["dout"])
    lens = g["lens"].tolist()
    scale, causal = float(g["scale"]), bool(g["causal"])
    for b in range(q.shape[0]):
        dq, dk, dv = orc.attention_backward_one(q[b], k[b, : lens[b]], v[b, : lens[b]], dout[b], scale, causal)
        torch.testing.assert_close(dq, t(g["dq"])[b], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(dk, t(g["dk"])[b, : lens[b]], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(dv, t(g["dv"])[b, : lens[b]], atol=1e-5, rtol=1e-4)
        assert t(g["dk"])[b, lens[b]:].abs().max().item() == 0 if lens[b] < k.shape[1] else True


@pytest.mark.parametrize("name", SPLIT_CASES)
def test_split_partials_and_combine_reproduce_split_reference(name):
    g = load_golden(name)
    q, k, v = t(g["q"]), t(g["k"]), t(g["v"])
    lens = g["lens"].tolist()
    scale, causal, splits = float(g["scale"]), bool(g["causal"]), int(g["splits"])
    for b in range(q.shape[0]):
        o_acc, l_acc = orc.split_partials(q[b], k[b, : lens[b]], v[b, : lens[b]], scale, causal, splits)
        n, h, sq, d = o_acc.shape
        out, lse = orc.combine(o_acc.reshape(n, h * sq, d), l_acc.reshape(n, h * sq))
        torch.testing.assert_close(out.view(h, sq, d).transpose(0, 1), t(g["out"])[b], atol=2e-6, rtol=1e-5)
        torch.testing.assert_close(lse.view(h, sq), _normalise_lse(t(g["lse"])[b]), atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("name,paged", [("cache_contiguous", False), ("cache_paged", True)])
def test_cache_append_and_gather(name, paged):
    g = load_golden(name)
    k_cache, v_cache = t(g["k_cache_before"]).clone(), t(g["v_cache_before"]).clone()
    lens = t(g["lens"])
    idx = None if paged else t(g["cache_batch_idx"])
    table = t(g["block_table"]) if paged else None
    orc.cache_append(k_cache, v_cache, t(g["k_new"]), t(g["v_new"]), lens, idx, table)
    assert torch.equal(k_cache, t(g["k_cache_after"]))  # bit-exact: pure copies
    assert torch.equal(v_cache, t(g["v_cache_after"]))
    ends = (lens + g["k_new"].shape[1]).tolist()
    ks, vs = orc.cache_gather(k_cache, v_cache, ends, idx, table)
    for b, n in enumerate(ends):
        assert torch.equal(ks[b], t(g["k_used"])[b, :n])
        assert torch.equal(vs[b], t(g["v_used"])[b, :n])


def test_dead_rows_follow_kernel_convention():
    # causal with more queries than keys: the first rows see nothing -> O = 0 and LSE = 0
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(1, 6, 2, 64, generator=gen).half()
    k = torch.randn(1, 2, 2, 64, generator=gen).half()
    v = torch.randn(1, 2, 2, 64, generator=gen).half()
    out, lse = orc.attention_forward(q, k, v, None, True)
    assert out[0, :4].abs().max().item() == 0 and lse[0, :, :4].abs().max().item() == 0
    assert out[0, 4:].abs().max().item() > 0
