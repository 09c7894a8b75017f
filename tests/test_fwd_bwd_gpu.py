"""GPU parity of the forward and backward kernels against the CPU fp32 oracle, through the torch
binding (which calls the C ABI).  Shapes follow the reference's grid (test_flash_attn.py:51-140 of
Cy-47/flash-attention-turing: odd lengths, Sq != Sk both ways, GQA/MQA head pairs, both head dims,
causal on/off, explicit scale) plus MHA cases for the packed variants, which the reference's grid
never reaches (all of its head pairs have Hq != Hk)."""
import pytest
import torch

from helpers import (LSE_TOL, assert_reference_suite_bounds, assert_within_twice_reference_kernel,
                     emulate_reference_kernel, emulate_reference_kernel_one, emulate_reference_kernel_varlen,
                     err_stats, load_golden, randn_half, t)
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"

SEQ_PAIRS = [(1, 1), (2, 2), (63, 65), (65, 63), (127, 129), (128, 128), (129, 257), (257, 129), (113, 203),
             (256, 512), (512, 256), (384, 384), (897, 1024), (1025, 1023), (1, 239), (239, 1), (799, 3), (3, 799)]
HEAD_PAIRS = [(2, 1), (4, 2), (6, 3), (6, 1), (4, 4)]


def _inputs(seed, b, sq, sk, h, hk, d):
    gen = torch.Generator().manual_seed(seed)
    return (randn_half(gen, b, sq, h, d), randn_half(gen, b, sk, hk, d), randn_half(gen, b, sk, hk, d),
            randn_half(gen, b, sq, h, d))


def _check(name, got, want, emul, absolute=True):
    """The stated tolerance: error against the fp32 oracle within twice the error of the reference's CUDA
    kernel on the same inputs (emulated rounding points, helpers.py).  ``absolute`` adds the reference
    suite's own bounds (max 9e-3, mean 2e-4), which are meant for its grid of short sequences: at the
    benchmark sizes |dK|, |dV| reach 16 and more, where half an fp16 ulp of the result alone is 8e-3."""
    assert_within_twice_reference_kernel(name, got, want, emul)
    if absolute:
        assert_reference_suite_bounds(name, got, want, emul)


@pytest.fixture
def single_kernel_backward(ext):
    """Runs the test body with the single-kernel backward selected, and puts the default back afterwards."""
    ext.set_single_kernel_backward(True)
    yield
    ext.set_single_kernel_backward(False)


@pytest.mark.parametrize("path", ["single_kernel", "two_kernels"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", SEQ_PAIRS)
def test_dense_forward_backward_grid(ext, request, d, causal, sq, sk, path):
    from flash_attention_turing_b200 import flash_attn_func

    if path == "single_kernel":
        request.getfixturevalue("single_kernel_backward")

    idx = SEQ_PAIRS.index((sq, sk))
    h, hk = HEAD_PAIRS[idx % len(HEAD_PAIRS)]
    b = 1 + idx % 3
    scale = None if idx % 2 == 0 else 0.3
    q, k, v, dout = _inputs(100 + idx, b, sq, sk, h, hk, d)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = flash_attn_func(qd, kd, vd, softmax_scale=scale, causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), dout.to(DEV))
    s = d ** -0.5 if scale is None else scale
    o_ref, _ = orc.attention_forward(q, k, v, s, causal)
    rq, rk, rv = orc.attention_backward(q, k, v, dout, s, causal)
    em = emulate_reference_kernel(q, k, v, dout, s, causal)
    _check("O", out, o_ref, em.out)
    _check("dQ", dq, rq, em.dq)
    _check("dK", dk, rk, em.dk)
    _check("dV", dv, rv, em.dv)


def test_c1_forward_full_size(ext):
    # C1 of the benchmark configs: forward, non-causal, B2 S512 H8 D64, scale 1/sqrt(64); O and LSE of
    # every (batch, head) against the oracle.
    b, s, h, d = 2, 512, 8, 64
    q, k, v, _ = _inputs(1001, b, s, s, h, h, d)
    out, lse = ext.fwd(q.to(DEV), k.to(DEV), v.to(DEV), d ** -0.5, False)
    o_ref, lse_ref = orc.attention_forward(q, k, v, None, False)
    em = emulate_reference_kernel(q, k, v, None, d ** -0.5, False)
    _check("O", out, o_ref, em.out)
    assert err_stats(lse, lse_ref)[0] <= LSE_TOL


@pytest.mark.parametrize("name", ["fwd_d64_noncausal", "fwd_d64_causal", "fwd_d128_causal_gqa", "fwd_d128_sq_gt_sk"])
def test_golden_fixtures(ext, name):
    # fixtures hold outputs of the reference's own Python math; keys beyond lens[b] are cut per sequence
    g = load_golden(name)
    q, k, v, dout = (t(g[x]) for x in ("q", "k", "v", "dout"))
    lens = g["lens"].tolist()
    scale, causal = float(g["scale"]), bool(g["causal"])
    for b in range(q.shape[0]):
        qb, kb, vb = q[b:b + 1].to(DEV), k[b:b + 1, : lens[b]].contiguous().to(DEV), v[b:b + 1, : lens[b]].contiguous().to(DEV)
        out, lse = ext.fwd(qb, kb, vb, scale, causal)
        dq, dk, dv = ext.bwd(qb, kb, vb, out, lse, dout[b:b + 1].to(DEV), scale, causal)
        want_out = torch.nan_to_num(t(g["out"])[b:b + 1], nan=0.0)
        want_lse = t(g["lse"])[b:b + 1]
        want_lse = torch.where(torch.isfinite(want_lse), want_lse, torch.zeros_like(want_lse))
        em = emulate_reference_kernel(q[b:b + 1], k[b:b + 1, : lens[b]], v[b:b + 1, : lens[b]], dout[b:b + 1], scale, causal)
        _check("O", out, want_out, em.out)
        assert err_stats(lse, want_lse)[0] <= LSE_TOL
        _check("dQ", dq, t(g["dq"])[b:b + 1], em.dq)
        _check("dK", dk, t(g["dk"])[b:b + 1, : lens[b]], em.dk)
        _check("dV", dv, t(g["dv"])[b:b + 1, : lens[b]], em.dv)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_packed_variants_match_unpacked(ext, d, causal):
    from flash_attention_turing_b200 import flash_attn_func, flash_attn_kvpacked_func, flash_attn_qkvpacked_func

    b, s, h = 2, 200, 4
    gen = torch.Generator().manual_seed(7 + d)
    qkv = randn_half(gen, b, s, 3, h, d).to(DEV).requires_grad_(True)
    dout = randn_half(gen, b, s, h, d).to(DEV)
    out_p = flash_attn_qkvpacked_func(qkv, causal=causal)
    (dqkv,) = torch.autograd.grad(out_p, qkv, dout)
    q, k, v = (qkv.detach()[:, :, i].contiguous().requires_grad_(True) for i in range(3))
    out = flash_attn_func(q, k, v, causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    assert torch.equal(out_p, out)  # same kernel, same data, strided vs contiguous: bit-identical
    assert torch.equal(dqkv[:, :, 0], dq) and torch.equal(dqkv[:, :, 1], dk) and torch.equal(dqkv[:, :, 2], dv)
    o_ref, _ = orc.attention_forward(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), None, causal)
    em = emulate_reference_kernel(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), None, d ** -0.5, causal)
    _check("O", out_p, o_ref, em.out)

    hk = 2
    kv = randn_half(gen, b, s, 2, hk, d).to(DEV).requires_grad_(True)
    q2 = q.detach().clone().requires_grad_(True)
    out_kv = flash_attn_kvpacked_func(q2, kv, causal=causal)
    dq2, dkv = torch.autograd.grad(out_kv, (q2, kv), dout)
    k2, v2 = (kv.detach()[:, :, i].contiguous().requires_grad_(True) for i in range(2))
    q3 = q.detach().clone().requires_grad_(True)
    out3 = flash_attn_func(q3, k2, v2, causal=causal)
    dq3, dk3, dv3 = torch.autograd.grad(out3, (q3, k2, v2), dout)
    assert torch.equal(out_kv, out3) and torch.equal(dq2, dq3)
    assert torch.equal(dkv[:, :, 0], dk3) and torch.equal(dkv[:, :, 1], dv3)


def test_bwd_binding_writes_into_given_strided_gradients(ext):
    b, s, h, d = 1, 130, 2, 64
    gen = torch.Generator().manual_seed(21)
    q, k, v, dout = (randn_half(gen, b, s, h, d).to(DEV) for _ in range(4))
    out, lse = ext.fwd(q, k, v, d ** -0.5, True)
    dq, dk, dv = ext.bwd(q, k, v, out, lse, dout, d ** -0.5, True)  # the reference's eight arguments
    packed = torch.full((b, s, 3, h, d), float("nan"), dtype=torch.half, device=DEV)
    views = packed.unbind(2)
    got = ext.bwd(q, k, v, out, lse, dout, d ** -0.5, True, *views)
    assert all(g.data_ptr() == w.data_ptr() for g, w in zip(got, views))  # written in place, nothing new
    assert torch.equal(packed[:, :, 0], dq) and torch.equal(packed[:, :, 1], dk) and torch.equal(packed[:, :, 2], dv)
    with pytest.raises(RuntimeError, match="shape"):
        ext.bwd(q, k, v, out, lse, dout, d ** -0.5, True, packed[:, :-1, 0], views[1], views[2])
    with pytest.raises(RuntimeError, match="float16"):
        ext.bwd(q, k, v, out, lse, dout, d ** -0.5, True, views[0].float(), views[1], views[2])


def _varlen_case(seed, lens_q, lens_k, h, hk, d):
    gen = torch.Generator().manual_seed(seed)
    cq = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32)
    ck = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32)
    tq, tk = int(cq[-1]), int(ck[-1])
    return (randn_half(gen, tq, h, d), randn_half(gen, tk, hk, d), randn_half(gen, tk, hk, d),
            randn_half(gen, tq, h, d), cq, ck)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lens_q,lens_k,h,hk", [
    ([100, 300, 57], [100, 300, 57], 4, 2),
    ([128, 1, 513, 64], [200, 64, 513, 1], 2, 1),
    ([1, 2, 3, 129, 255], [7, 2, 300, 129, 1], 6, 3),
    ([640], [640], 4, 4),
])
@pytest.mark.parametrize("path", ["single_kernel", "two_kernels"])
def test_varlen_forward_backward(ext, request, d, causal, lens_q, lens_k, h, hk, path):
    from flash_attention_turing_b200 import flash_attn_varlen_func

    if path == "single_kernel":
        request.getfixturevalue("single_kernel_backward")

    q, k, v, dout, cq, ck = _varlen_case(31 + d, lens_q, lens_k, h, hk, d)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = flash_attn_varlen_func(qd, kd, vd, cq.to(DEV), ck.to(DEV), max(lens_q), max(lens_k), causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), dout.to(DEV))
    o_ref, lses = orc.varlen_forward(q, k, v, cq, ck, None, causal)
    rq, rk, rv = orc.varlen_backward(q, k, v, dout, cq, ck, None, causal)
    em = emulate_reference_kernel_varlen(q, k, v, dout, cq, ck, d ** -0.5, causal)
    _check("O", out, o_ref, em.out)
    _check("dQ", dq, rq, em.dq)
    _check("dK", dk, rk, em.dk)
    _check("dV", dv, rv, em.dv)
    # padded LSE (b, h, max_seqlen_q): valid part matches, padding stays zero
    _, lse = ext.varlen_fwd(qd.detach(), kd.detach(), vd.detach(), cq.to(DEV), ck.to(DEV), max(lens_q), max(lens_k),
                            d ** -0.5, causal)
    for i, l in enumerate(lses):
        assert err_stats(lse[i, :, : lens_q[i]], l)[0] <= LSE_TOL
        assert lse[i, :, lens_q[i]:].abs().max().item() == 0 if lens_q[i] < max(lens_q) else True


def test_varlen_packed_variants(ext):
    from flash_attention_turing_b200 import (flash_attn_varlen_func, flash_attn_varlen_kvpacked_func,
                                             flash_attn_varlen_qkvpacked_func)

    lens = [90, 257, 33]
    d, h = 128, 4
    gen = torch.Generator().manual_seed(5)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32).to(DEV)
    total = sum(lens)
    qkv = randn_half(gen, total, 3, h, d).to(DEV).requires_grad_(True)
    dout = randn_half(gen, total, h, d).to(DEV)
    out_p = flash_attn_varlen_qkvpacked_func(qkv, cu, max(lens), causal=True)
    (dqkv,) = torch.autograd.grad(out_p, qkv, dout)
    q, k, v = (qkv.detach()[:, i].contiguous().requires_grad_(True) for i in range(3))
    out = flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    assert torch.equal(out_p, out)
    assert torch.equal(dqkv[:, 0], dq) and torch.equal(dqkv[:, 1], dk) and torch.equal(dqkv[:, 2], dv)
    kv = torch.stack((k.detach(), v.detach()), dim=1).requires_grad_(True)
    q2 = q.detach().clone().requires_grad_(True)
    out_kv = flash_attn_varlen_kvpacked_func(q2, kv, cu, cu, max(lens), max(lens), causal=True)
    dq2, dkv = torch.autograd.grad(out_kv, (q2, kv), dout)
    assert torch.equal(out_kv, out) and torch.equal(dq2, dq) and torch.equal(dkv[:, 0], dk) and torch.equal(dkv[:, 1], dv)


def test_run_to_run_determinism(ext):
    # Two-kernel backward (the default): every accumulation order is fixed (no atomics), so repeated launches are
    # bit-identical, which also catches races on shared memory / TMEM.  Single-kernel backward: O, LSE, dK, dV
    # are bit-identical as well; dQ is summed with global fp32 reductions in scheduling order, so it is only
    # held to agree within one fp16 ulp of its largest value from run to run.
    q, k, v, dout = _inputs(77, 2, 700, 700, 4, 2, 128)
    qd, kd, vd, dd = (x.to(DEV) for x in (q, k, v, dout))
    for single in (False, True):
        ext.set_single_kernel_backward(single)
        try:
            first = None
            for _ in range(3):
                out, lse = ext.fwd(qd, kd, vd, 128 ** -0.5, True)
                dq, dk, dv = ext.bwd(qd, kd, vd, out, lse, dd, 128 ** -0.5, True)
                cur = [out, lse, dk, dv, dq]
                if first is None:
                    first = [x.clone() for x in cur]
                    continue
                assert all(torch.equal(a, b) for a, b in zip(first[:4], cur[:4]))
                if not single:
                    assert torch.equal(first[4], dq)
                else:
                    ulp = 2.0 ** -10 * first[4].float().abs().max().item()
                    assert (first[4].float() - dq.float()).abs().max().item() <= ulp
        finally:
            ext.set_single_kernel_backward(False)


@pytest.mark.parametrize("d", [64, 128])
def test_both_backward_paths_agree(ext, d):
    # the single-kernel and the two-kernel backward compute the same sums with the same rounding points:
    # dK and dV agree bit for bit or within an ulp (different accumulation chunks), dQ within an ulp
    q, k, v, dout = _inputs(78, 2, 600, 900, 6, 2, d)
    qd, kd, vd, dd = (x.to(DEV) for x in (q, k, v, dout))
    out, lse = ext.fwd(qd, kd, vd, d ** -0.5, True)
    a = ext.bwd(qd, kd, vd, out, lse, dd, d ** -0.5, True)
    ext.set_single_kernel_backward(True)
    try:
        b = ext.bwd(qd, kd, vd, out, lse, dd, d ** -0.5, True)
    finally:
        ext.set_single_kernel_backward(False)
    for x, y in zip(a, b):
        assert (x.float() - y.float()).abs().max().item() <= 2.0 ** -9 * max(1.0, y.float().abs().max().item())


def test_no_grad_and_requires_grad_flags(ext):
    from flash_attention_turing_b200 import flash_attn_func

    q, k, v, _ = _inputs(3, 1, 64, 64, 2, 2, 64)
    with torch.no_grad():
        out = flash_attn_func(q.to(DEV), k.to(DEV), v.to(DEV))
    assert not out.requires_grad
    qd = q.to(DEV).requires_grad_(True)
    out = flash_attn_func(qd, k.to(DEV), v.to(DEV), causal=True)
    (dq,) = torch.autograd.grad(out.float().sum(), qd)
    assert dq.shape == qd.shape and dq.dtype == torch.float16


def test_binding_errors(ext):
    q = torch.randn(1, 8, 4, 96, device=DEV, dtype=torch.half)
    with pytest.raises(RuntimeError, match="head_dim 64 or 128"):
        ext.fwd(q, q, q, 1.0, False)
    q = torch.randn(1, 8, 4, 64, device=DEV, dtype=torch.half)
    k = torch.randn(1, 8, 3, 64, device=DEV, dtype=torch.half)
    with pytest.raises(RuntimeError, match="divisible by num_heads_k"):
        ext.fwd(q, k, k, 1.0, False)
    with pytest.raises(RuntimeError, match="rank-4"):
        ext.fwd(q[0], k[0], k[0], 1.0, False)


def _sampled_slices_check(q, k, v, dout, out, lse, dq, dk, dv, slices, causal=True):
    """Attention is independent per (batch, head): a slice of a full-size launch must match the oracle of
    that slice, within twice the reference kernel's error (emulated on the same slice)."""
    d = q.shape[-1]
    for bi, hi in slices:
        sl = lambda x: x[bi:bi + 1, :, hi:hi + 1].cpu()  # noqa: E731
        o_ref, lse_ref = orc.attention_forward(sl(q), sl(k), sl(v), None, causal)
        rq, rk, rv = orc.attention_backward(sl(q), sl(k), sl(v), sl(dout), None, causal)
        em = emulate_reference_kernel(sl(q), sl(k), sl(v), sl(dout), d ** -0.5, causal)
        _check("O", sl(out), o_ref, em.out, absolute=False)
        assert err_stats(lse[bi:bi + 1, hi:hi + 1], lse_ref)[0] <= LSE_TOL
        _check("dQ", sl(dq), rq, em.dq, absolute=False)
        _check("dK", sl(dk), rk, em.dk, absolute=False)
        _check("dV", sl(dv), rv, em.dv, absolute=False)


@pytest.mark.parametrize("s", [4096, 8192])
def test_full_size_causal_config_by_sampling(ext, s):
    # S = 4096: C2 of the benchmark configs (B4 S4096 H32 D128 causal, forward + backward).  S = 8192: the
    # shape the headline metric is quoted on.  Full-size launches; the oracle is evaluated on two
    # (batch, head) slices.
    b, h, d = 4, 32, 128
    gen = torch.Generator(device=DEV).manual_seed(1002)
    q, k, v, dout = (torch.randn(b, s, h, d, device=DEV, dtype=torch.half, generator=gen) for _ in range(4))
    out, lse = ext.fwd(q, k, v, d ** -0.5, True)
    dq, dk, dv = ext.bwd(q, k, v, out, lse, dout, d ** -0.5, True)
    _sampled_slices_check(q, k, v, dout, out, lse, dq, dk, dv, [(0, 0), (3, 17)])
    # size-independent property: every softmax row sums to one => with V = 1, O = 1 exactly
    ones = torch.ones_like(v)
    o1, _ = ext.fwd(q, k, ones, d ** -0.5, True)
    assert (o1.float() - 1).abs().max().item() <= 2e-3


def _c3_lengths():
    """C3 of the benchmark configs: 16 sequences, lengths U[256, 4096] (seeded), capped at 32768 tokens."""
    gen = torch.Generator().manual_seed(1003)
    lens = torch.randint(256, 4097, (16,), generator=gen)
    total = int(lens.sum())
    if total > 32768:
        lens = torch.clamp(lens * 32768 // total, min=256)
    return [int(x) for x in lens]


def test_c3_gqa_varlen_full_size(ext):
    # C3: GQA varlen forward + backward, causal, Hq32 Hkv8 D128, 16 sequences.  The full-size launch is
    # checked on two whole sequences (all heads of one KV group each) against the oracle.
    from flash_attention_turing_b200 import flash_attn_varlen_func

    lens = _c3_lengths()
    assert sum(lens) <= 32768
    h, hk, d = 32, 8, 128
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    total = int(cu[-1])
    gen = torch.Generator(device=DEV).manual_seed(1003)
    q = torch.randn(total, h, d, device=DEV, dtype=torch.half, generator=gen).requires_grad_(True)
    k = torch.randn(total, hk, d, device=DEV, dtype=torch.half, generator=gen).requires_grad_(True)
    v = torch.randn(total, hk, d, device=DEV, dtype=torch.half, generator=gen).requires_grad_(True)
    dout = torch.randn(total, h, d, device=DEV, dtype=torch.half, generator=gen)
    out = flash_attn_varlen_func(q, k, v, cu.to(DEV), cu.to(DEV), max(lens), max(lens), causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    order = sorted(range(16), key=lambda i: lens[i])
    for seq, kv_head in ((order[0], 0), (order[8], 5)):
        a, b = int(cu[seq]), int(cu[seq + 1])
        hs = slice(kv_head * 4, kv_head * 4 + 4)
        qs, ks, vs, ds = (x.detach()[a:b].cpu() for x in (q[:, hs], k[:, kv_head:kv_head + 1], v[:, kv_head:kv_head + 1], dout[:, hs]))
        o_ref, _ = orc.attention_forward_one(qs, ks, vs, d ** -0.5, True)
        rq, rk, rv = orc.attention_backward_one(qs, ks, vs, ds, d ** -0.5, True)
        em = emulate_reference_kernel_one(qs, ks, vs, ds, d ** -0.5, True)
        _check("O", out[a:b, hs], o_ref, em.out, absolute=False)
        _check("dQ", dq[a:b, hs], rq, em.dq, absolute=False)
        _check("dK", dk[a:b, kv_head:kv_head + 1], rk, em.dk, absolute=False)
        _check("dV", dv[a:b, kv_head:kv_head + 1], rv, em.dv, absolute=False)


@pytest.mark.parametrize("d", [64, 128])
def test_c5_long_context_by_sampling(ext, d):
    # C5: B1 S65536 H16 causal, forward + backward at full size on a head shard (2 of 16 heads, as one rank
    # of an 8-GPU head-sharded run).  Causality makes exact value checks of the 65536-token launch cheap:
    #   * rows [0, 8192) of O, LSE and dQ depend only on the first 8192 tokens: they must equal the oracle of
    #     that prefix;
    #   * dK, dV of the keys [61440, 65536) receive contributions from the query rows >= 61440 only: they must
    #     equal the oracle evaluated on those 4096 query rows against all keys.
    # Both within twice the reference kernel's (emulated) error; sampled rows and two identities on top.
    b, s, h = 1, 65536, 2
    scale = d ** -0.5
    gen = torch.Generator(device=DEV).manual_seed(1005)
    q, k, v, dout = (torch.randn(b, s, h, d, device=DEV, dtype=torch.half, generator=gen) for _ in range(4))
    out, lse = ext.fwd(q, k, v, scale, True)
    rows = [0, 1, 127, 128, 4095, 30000, 65535]
    for r in rows:
        qs = q[:, r:r + 1, :1].cpu()
        o_ref, lse_ref = orc.attention_forward(qs, k[:, : r + 1, :1].cpu(), v[:, : r + 1, :1].cpu(), None, False)
        assert err_stats(out[:, r:r + 1, :1], o_ref)[0] <= 2e-3
        assert err_stats(lse[:, :1, r:r + 1], lse_ref)[0] <= LSE_TOL
    o1, _ = ext.fwd(q, k, torch.ones_like(v), scale, True)
    assert (o1.float() - 1).abs().max().item() <= 2e-3
    dq, dk, dv = ext.bwd(q, k, v, out, lse, dout, scale, True)
    assert not any(torch.isnan(x).any().item() for x in (dq, dk, dv))
    hd = 1  # the head that is compared value by value
    one = lambda x, a, e: x[0, a:e, hd:hd + 1].cpu()  # noqa: E731
    # prefix: the first 8192 tokens
    n = 8192
    qp, kp, vp, dp = (one(x, 0, n) for x in (q, k, v, dout))
    o_ref, lse_ref = orc.attention_forward_one(qp, kp, vp, scale, True)
    rq, _, _ = orc.attention_backward_one(qp, kp, vp, dp, scale, True)
    em = emulate_reference_kernel_one(qp, kp, vp, dp, scale, True)
    _check("O[:8192]", one(out, 0, n), o_ref, em.out, absolute=False)
    assert err_stats(lse[0, hd:hd + 1, :n], lse_ref)[0] <= LSE_TOL
    _check("dQ[:8192]", one(dq, 0, n), rq, em.dq, absolute=False)
    # tail: the last 4096 query rows against all keys
    r0 = s - 4096
    qa, ka, va, da = (one(x, 0, s) for x in (q, k, v, dout))
    rq, rk, rv = orc.attention_backward_one(qa, ka, va, da, scale, True, row_chunk=1024, row_start=r0)
    em = emulate_reference_kernel_one(qa, ka, va, da, scale, True, row_chunk=1024, row_start=r0)
    _check("dQ[-4096:]", one(dq, r0, s), rq[r0:], em.dq[r0:], absolute=False)
    _check("dK[-4096:]", one(dk, r0, s), rk[r0:], em.dk[r0:], absolute=False)
    _check("dV[-4096:]", one(dv, r0, s), rv[r0:], em.dv[r0:], absolute=False)
    # identities over the whole launch: sum(dQ * Q) = sum(dK * K) (the scores depend on Q K^T only) ...
    lhs = (dq.float() * q.float()).sum().item()
    rhs = (dk.float() * k.float()).sum().item()
    assert abs(lhs - rhs) <= 2e-3 * max(abs(lhs), abs(rhs), (dq.float().abs() * q.float().abs()).sum().item() * 1e-3)
    # ... and dV of the last key row is exactly P[last query, last key] * dO[last query]
    p_last = torch.exp((q[0, -1].float() * k[0, -1].float()).sum(-1) * scale - lse[0, :, -1])
    want = p_last[:, None] * dout[0, -1].float()
    assert (dv[0, -1].float() - want).abs().max().item() <= 1e-3


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lens,h,hk,d,poison", [([100, 300, 57], 4, 2, 128, 1), ([200, 64, 513], 2, 1, 64, 2),
                                                ([130, 130, 130], 2, 2, 128, 0)])
def test_varlen_gradients_ignore_nan_in_a_neighbouring_sequence(ext, lens, h, hk, d, poison, causal):
    """The sequences of a packed batch are independent: NaN in every tensor of one sequence must not reach the
    outputs or gradients of the others (rows of the next sequence share 128-row tiles with this one)."""
    from flash_attention_turing_b200 import flash_attn_varlen_func

    gen = torch.Generator().manual_seed(5)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    total = int(cu[-1])
    q, do = randn_half(gen, total, h, d), randn_half(gen, total, h, d)
    k, v = randn_half(gen, total, hk, d), randn_half(gen, total, hk, d)
    ro, _ = orc.varlen_forward(q, k, v, cu, cu, None, causal)
    rq, rk, rv = orc.varlen_backward(q, k, v, do, cu, cu, None, causal)
    em = emulate_reference_kernel_varlen(q, k, v, do, cu, cu, d ** -0.5, causal)
    lo, hi = int(cu[poison]), int(cu[poison + 1])
    for t in (q, k, v, do):
        t[lo:hi] = float("nan")
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = flash_attn_varlen_func(qd, kd, vd, cu.to(DEV), cu.to(DEV), max(lens), max(lens), causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do.to(DEV))
    keep = torch.ones(total, dtype=torch.bool)
    keep[lo:hi] = False
    for name, got, want, emu in (("O", out, ro, em.out), ("dQ", dq, rq, em.dq), ("dK", dk, rk, em.dk), ("dV", dv, rv, em.dv)):
        got = got.detach().float().cpu()[keep]
        assert not torch.isnan(got).any(), name
        _check(name, got, want[keep], emu[keep])


CANARY = 0x7BCD  # an fp16 bit pattern (finite, 6.2e4) that no kernel result takes by accident


def _canary_view(shape, pad_elems=4096, dtype=torch.half):
    """A tensor of `shape` cut out of a larger canary-filled buffer: `pad_elems` untouched elements before and
    after, and a row pitch one head wider than needed, so that every (row) has a gap after its last head.
    Returns (view, buffer, mask of the elements the view covers)."""
    b, s, h, d = shape
    pitch = (h + 1) * d
    n = b * s * pitch
    buf = torch.empty(n + 2 * pad_elems, dtype=dtype, device=DEV)
    if dtype == torch.half:
        buf.view(torch.int16).fill_(CANARY)
    else:
        buf.view(torch.int32).fill_(0x7BCD7BCD)
    view = buf[pad_elems:pad_elems + n].view(b, s, h + 1, d)[:, :, :h]
    mask = torch.zeros_like(buf, dtype=torch.bool)
    mask[pad_elems:pad_elems + n].view(b, s, h + 1, d)[:, :, :h] = True
    return view, buf, mask


def _canaries_intact(buf, mask):
    raw = buf.view(torch.int16) if buf.dtype == torch.half else buf.view(torch.int32)
    want = CANARY if buf.dtype == torch.half else 0x7BCD7BCD
    return bool((raw[~mask] == want).all().item())


@pytest.mark.parametrize("flags", [0, 1])  # 0: two-kernel backward, 1: FA_BWD_SINGLE_KERNEL
@pytest.mark.parametrize("b,sq,sk,h,hk,d,causal", [(2, 129, 257, 4, 2, 64, True), (1, 385, 131, 3, 1, 128, False),
                                                   (2, 1, 300, 2, 2, 128, True), (1, 700, 700, 6, 3, 64, True)])
def test_guard_bands_around_outputs_and_scratch(b, sq, sk, h, hk, d, causal, flags):
    """Nothing is written outside the tensors the caller handed over: O, LSE, dQ, dK, dV and the backward
    scratch are cut out of canary-filled buffers (pads before and after, a gap after every row) through the
    C ABI's strides, and the canaries are intact after forward and backward at odd sizes.  (The memory
    checker of the CUDA toolkit is not available on the test machines.)"""
    import ctypes

    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q, k, v, dout = (x.to(DEV) for x in _inputs(5 + sq, b, sq, sk, h, hk, d))
    o, o_buf, o_mask = _canary_view((b, sq, h, d))
    dq, dq_buf, dq_mask = _canary_view((b, sq, h, d))
    dk, dk_buf, dk_mask = _canary_view((b, sk, hk, d))
    dv, dv_buf, dv_mask = _canary_view((b, sk, hk, d))
    lse_buf = torch.empty(b * h * sq + 2048, dtype=torch.float32, device=DEV)
    lse_buf.view(torch.int32).fill_(0x7BCD7BCD)
    lse = lse_buf[1024:1024 + b * h * sq].view(b, h, sq)
    scale = d ** -0.5
    capi.check(lib.fa_fwd(ctypes.byref(capi.fwd_params(q, k, v, o, lse, scale, causal)), stream))
    bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, None, scale, causal)
    bp.flags = flags
    need = lib.fa_bwd_workspace_bytes(ctypes.byref(bp))
    ws_buf = torch.empty(need + 8192, dtype=torch.uint8, device=DEV)
    ws_buf.fill_(0xA5)
    bp.workspace, bp.workspace_bytes = ws_buf.data_ptr() + 4096, need
    capi.check(lib.fa_bwd(ctypes.byref(bp), stream))
    torch.cuda.synchronize()
    for name, buf, mask in (("O", o_buf, o_mask), ("dQ", dq_buf, dq_mask), ("dK", dk_buf, dk_mask), ("dV", dv_buf, dv_mask)):
        assert _canaries_intact(buf, mask), f"{name}: a write outside the tensor"
    raw = lse_buf.view(torch.int32)
    assert bool((raw[:1024] == 0x7BCD7BCD).all()) and bool((raw[1024 + b * h * sq:] == 0x7BCD7BCD).all()), "LSE"
    assert bool((ws_buf[:4096] == 0xA5).all()) and bool((ws_buf[4096 + need:] == 0xA5).all()), "backward scratch"
    # and the results inside are the right ones
    qc, kc, vc, dc = (x.cpu() for x in (q, k, v, dout))
    o_ref, lse_ref = orc.attention_forward(qc, kc, vc, None, causal)
    rq, rk, rv = orc.attention_backward(qc, kc, vc, dc, None, causal)
    em = emulate_reference_kernel(qc, kc, vc, dc, scale, causal)
    for name, got, want, emu in (("O", o, o_ref, em.out), ("dQ", dq, rq, em.dq), ("dK", dk, rk, em.dk), ("dV", dv, rv, em.dv)):
        _check(name, got, want, emu)
    assert err_stats(lse, lse_ref)[0] <= LSE_TOL
    assert lib.fa_device_status(1) == 0


def _multi_wave_case(seed, causal=True, d=128):
    """More work items than SMs, so that the forward takes its items from the global work counter."""
    gen = torch.Generator().manual_seed(seed)
    b, s, h, hk = 2, 2048, 12, 4   # 2 x 12 x 8 = 192 items of 256 rows
    q, k, v = randn_half(gen, b, s, h, d), randn_half(gen, b, s, hk, d), randn_half(gen, b, s, hk, d)
    return q.to(DEV), k.to(DEV), v.to(DEV), d ** -0.5, causal


def test_forward_work_counters_are_left_clean_over_many_launches(ext):
    """The persistent forward takes a {next item, finished CTAs} pair from a pool of 1024 and its last CTA puts
    the pair back to zero.  2200 launches go round the pool twice: a pair left dirty by an earlier launch would
    make a later one skip items, i.e. leave rows of O unwritten."""
    q, k, v, scale, causal = _multi_wave_case(31)
    want, want_lse = ext.fwd(q, k, v, scale, causal)
    out, lse = torch.empty_like(want), torch.empty_like(want_lse)
    for i in range(2200):
        if i % 550 == 0:
            out.fill_(float("nan"))
        ext.fwd(q, k, v, scale, causal, out=out, lse=lse)
        if i % 550 == 549:
            assert torch.equal(out, want) and torch.equal(lse, want_lse), i
    assert ext.device_status(True) == 0


def test_forward_launches_on_two_streams_do_not_share_work_counters(ext):
    q, k, v, scale, causal = _multi_wave_case(32)
    q2, k2, v2, _, _ = _multi_wave_case(33, causal=False)
    want, _ = ext.fwd(q, k, v, scale, causal)
    want2, _ = ext.fwd(q2, k2, v2, scale, False)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(20):  # launches of the two streams overlap on the GPU (each fills it for ~30 us)
        with torch.cuda.stream(s1):
            o1, _ = ext.fwd(q, k, v, scale, causal)
        with torch.cuda.stream(s2):
            o2, _ = ext.fwd(q2, k2, v2, scale, False)
        outs.append((o1, o2))
    torch.cuda.synchronize()
    for o1, o2 in outs:
        assert torch.equal(o1, want) and torch.equal(o2, want2)
    assert ext.device_status(True) == 0


def test_forward_in_a_cuda_graph_replays(ext):
    """A captured launch keeps the counter pair it was given; it is clean again whenever a replay ends, so the
    graph can be replayed any number of times (new inputs written into the captured tensors)."""
    q, k, v, scale, causal = _multi_wave_case(34)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=DEV)
    ext.fwd(q, k, v, scale, causal, out=out, lse=lse)  # first launch on this device outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ext.fwd(q, k, v, scale, causal, out=out, lse=lse)
    gen = torch.Generator().manual_seed(35)
    for _ in range(5):
        q.copy_(randn_half(gen, *q.shape))
        graph.replay()
        got = out.clone()
        want, _ = ext.fwd(q, k, v, scale, causal)
        assert torch.equal(got, want)
    assert ext.device_status(True) == 0


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("h,hk,d", [(3, 1, 128), (4, 4, 64)])
def test_varlen_forward_many_ragged_sequences(ext, h, hk, d, causal):
    """The forward's work-item mapping for packed sequences (slots from cu_seqlens_q / 256) over 70 sequences with
    the lengths that matter to it: empty ones, single rows, exact multiples of 256 and of 128, one row more or
    less, and long ones -- more items than SMs, so that the counter path runs.  Every sequence must equal the
    dense launch on that sequence alone (same kernel, same rounding: bit for bit), which is compared with the
    oracle elsewhere; LSE padding stays zero."""
    gen = torch.Generator().manual_seed(77 + d)
    lens = [0, 1, 255, 256, 257, 511, 512, 513, 128, 127, 129, 0, 0, 3, 1024, 2047, 2048, 2049, 5, 640]
    lens += [int(x) for x in torch.randint(1, 700, (50,), generator=gen)]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    total = int(cu[-1])
    q, k, v = randn_half(gen, total, h, d).to(DEV), randn_half(gen, total, hk, d).to(DEV), randn_half(gen, total, hk, d).to(DEV)
    scale = d ** -0.5
    out, lse = ext.varlen_fwd(q, k, v, cu.to(DEV), cu.to(DEV), max(lens), max(lens), scale, causal)
    assert not torch.isnan(out).any()
    for i, n in enumerate(lens):
        a, b = int(cu[i]), int(cu[i + 1])
        if n == 0:
            assert lse[i].abs().max().item() == 0
            continue
        o1, l1 = ext.fwd(q[a:b].unsqueeze(0), k[a:b].unsqueeze(0), v[a:b].unsqueeze(0), scale, causal)
        assert torch.equal(out[a:b], o1[0]), (i, n)
        assert torch.equal(lse[i, :, :n], l1[0]), (i, n)
        assert lse[i, :, n:].abs().max().item() == 0 if n < max(lens) else True
    assert ext.device_status(True) == 0


def test_package_reports_the_device_status_word(ext):
    import flash_attention_turing_b200 as fa

    assert fa.device_status() == 0
    assert fa.device_status(reset=True) == 0
