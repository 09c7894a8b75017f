"""The reference's own test grid, run against this library's kernels on the GPU.

Cy-47/flash-attention-turing's test_flash_attn.py runs every distinct (seqlen_q, seqlen_k) pair of its
SEQLEN_CASES (:59-140) with every head pair of NHEAD_PAIRS (:57), batch sizes 1 and 3 (:53), softmax scales
None and 0.3 (:54), both head dims and causal on / off, through the dense (:703-775), kv-packed (:778-855),
qkv-packed (:857-932) and varlen (:935-1101, lengths from the generator of :393-464) entry points, and the
KV-cache path with randomised lengths (:1387-1488).  The same grid runs here; the MHA pair (4, 4) is added
because the reference's grid never reaches Hq == Hk.

Two bounds are asserted on O, dQ, dK, dV of every case:
  * the tolerance stated for this operator -- max (and mean) absolute error against the fp32 oracle within
    twice that of the reference's CUDA kernel, whose rounding points are emulated (helpers.py);
  * the reference suite's own absolute bounds (max 9e-3, mean 2e-4, test_flash_attn.py:42-49,250-257).
LSE within 1e-3.

The oracle and the emulation are evaluated on CUDA tensors here (strict fp32: TF32 is off), because the grid
has several thousand cases; test_oracle_on_device_matches_oracle_on_cpu ties that evaluation to the CPU one.
"""
import zlib

import pytest
import torch

from helpers import (LSE_TOL, assert_reference_suite_bounds, assert_within_twice_reference_kernel,
                     emulate_reference_kernel, emulate_reference_kernel_varlen, err_stats, randn_half)
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"

SEQ_PAIRS = [(1, 1), (1, 2), (1, 64), (1, 128), (1, 1024), (2, 1), (2, 2), (63, 63), (64, 1), (64, 2), (64, 64),
             (64, 65), (64, 128), (64, 129), (64, 256), (64, 257), (65, 64), (65, 65), (65, 128), (127, 63),
             (127, 127), (128, 1), (128, 64), (128, 65), (128, 127), (128, 128), (128, 129), (128, 256), (128, 257),
             (128, 1024), (128, 1025), (129, 64), (129, 65), (129, 128), (129, 129), (256, 64), (256, 128),
             (256, 1024), (256, 1025), (257, 64), (257, 128), (512, 128), (512, 1024), (768, 128), (897, 1024),
             (959, 1024), (960, 1024), (961, 1024), (1023, 1024), (1024, 1), (1024, 2), (1024, 128), (1024, 256),
             (1024, 897), (1024, 1023), (1024, 1024), (1024, 1025), (1025, 1024)]
HEAD_PAIRS = [(2, 1), (4, 2), (6, 3), (6, 1), (4, 4)]
BATCH_SIZES = [1, 3]
SCALES = [None, 0.3]


@pytest.fixture(autouse=True, scope="module")
def _strict_fp32():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old


def _seed(*key) -> int:
    return zlib.crc32(repr(key).encode())


def _check_all(got, want, emul, absolute=True):
    """got / want / emul: dicts name -> tensor."""
    for name in got:
        assert_within_twice_reference_kernel(name, got[name], want[name], emul[name])
        if absolute:
            assert_reference_suite_bounds(name, got[name], want[name], emul[name])


@pytest.mark.parametrize("scale", SCALES)
@pytest.mark.parametrize("b", BATCH_SIZES)
@pytest.mark.parametrize("h,hk", HEAD_PAIRS)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("sq,sk", SEQ_PAIRS)
def test_dense_grid(ext, sq, sk, d, causal, h, hk, b, scale):
    from flash_attention_turing_b200 import flash_attn_func

    gen = torch.Generator().manual_seed(_seed(sq, sk, d, causal, h, hk, b, scale))
    q, k, v, dout = (randn_half(gen, b, s, n, d).to(DEV) for s, n in ((sq, h), (sk, hk), (sk, hk), (sq, h)))
    qd, kd, vd = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = flash_attn_func(qd, kd, vd, softmax_scale=scale, causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), dout)
    _, lse = ext.fwd(q, k, v, d ** -0.5 if scale is None else scale, causal)
    s = d ** -0.5 if scale is None else scale
    o_ref, lse_ref = orc.attention_forward(q, k, v, s, causal)
    rq, rk, rv = orc.attention_backward(q, k, v, dout, s, causal)
    em = emulate_reference_kernel(q, k, v, dout, s, causal)
    _check_all(dict(O=out, dQ=dq, dK=dk, dV=dv), dict(O=o_ref, dQ=rq, dK=rk, dV=rv),
               dict(O=em.out, dQ=em.dq, dK=em.dk, dV=em.dv))
    assert err_stats(lse, lse_ref)[0] <= LSE_TOL


def _reference_varlen_lengths(b, max_q, max_k, seed):
    """Lengths as the reference's generator draws them (test_flash_attn.py:405-408): U[1, max] per sequence,
    one sequence forced to the maximum."""
    rng = torch.Generator().manual_seed(seed)
    lq = torch.randint(1, max_q + 1, (b,), generator=rng)
    lk = torch.randint(1, max_k + 1, (b,), generator=rng)
    lq[torch.randint(0, b, (1,), generator=rng).item()] = max_q
    lk[torch.randint(0, b, (1,), generator=rng).item()] = max_k
    return [int(x) for x in lq], [int(x) for x in lk]


@pytest.mark.parametrize("scale", SCALES)
@pytest.mark.parametrize("b", BATCH_SIZES)
@pytest.mark.parametrize("h,hk", [(2, 1), (6, 3), (6, 1), (4, 4)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("max_q,max_k", SEQ_PAIRS[::2])
def test_varlen_grid(ext, max_q, max_k, d, causal, h, hk, b, scale):
    from flash_attention_turing_b200 import flash_attn_varlen_func

    seed = _seed("varlen", max_q, max_k, d, causal, h, hk, b, scale)
    lens_q, lens_k = _reference_varlen_lengths(b, max_q, max_k, seed)
    cq = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32)
    ck = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32)
    gen = torch.Generator().manual_seed(seed + 1)
    tq, tk = int(cq[-1]), int(ck[-1])
    q, k, v, dout = (randn_half(gen, t, n, d).to(DEV) for t, n in ((tq, h), (tk, hk), (tk, hk), (tq, h)))
    qd, kd, vd = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = flash_attn_varlen_func(qd, kd, vd, cq.to(DEV), ck.to(DEV), max_q, max_k, softmax_scale=scale, causal=causal)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), dout)
    s = d ** -0.5 if scale is None else scale
    o_ref, lses = orc.varlen_forward(q, k, v, cq, ck, s, causal)
    rq, rk, rv = orc.varlen_backward(q, k, v, dout, cq, ck, s, causal)
    em = emulate_reference_kernel_varlen(q, k, v, dout, cq, ck, s, causal)
    _check_all(dict(O=out, dQ=dq, dK=dk, dV=dv), dict(O=o_ref, dQ=rq, dK=rk, dV=rv),
               dict(O=em.out, dQ=em.dq, dK=em.dk, dV=em.dv))
    _, lse = ext.varlen_fwd(q, k, v, cq.to(DEV), ck.to(DEV), max_q, max_k, s, causal)
    for i, l in enumerate(lses):
        assert err_stats(lse[i, :, : lens_q[i]], l)[0] <= LSE_TOL


@pytest.mark.parametrize("b", BATCH_SIZES)
@pytest.mark.parametrize("h,hk", [(4, 2), (6, 1), (4, 4)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("sq,sk", [(64, 128), (129, 129), (128, 1025), (1024, 897), (1, 1024), (1024, 2)])
def test_kvpacked_grid(ext, sq, sk, d, causal, h, hk, b):
    # kv-packed entry point (test_flash_attn.py:778-855): same kernels through strided views of one tensor
    from flash_attention_turing_b200 import flash_attn_kvpacked_func

    gen = torch.Generator().manual_seed(_seed("kv", sq, sk, d, causal, h, hk, b))
    q, dout = randn_half(gen, b, sq, h, d).to(DEV), randn_half(gen, b, sq, h, d).to(DEV)
    kv = randn_half(gen, b, sk, 2, hk, d).to(DEV)
    qd, kvd = q.clone().requires_grad_(True), kv.clone().requires_grad_(True)
    out = flash_attn_kvpacked_func(qd, kvd, causal=causal)
    dq, dkv = torch.autograd.grad(out, (qd, kvd), dout)
    k, v = kv[:, :, 0].contiguous(), kv[:, :, 1].contiguous()
    s = d ** -0.5
    o_ref, _ = orc.attention_forward(q, k, v, s, causal)
    rq, rk, rv = orc.attention_backward(q, k, v, dout, s, causal)
    em = emulate_reference_kernel(q, k, v, dout, s, causal)
    _check_all(dict(O=out, dQ=dq, dK=dkv[:, :, 0], dV=dkv[:, :, 1]), dict(O=o_ref, dQ=rq, dK=rk, dV=rv),
               dict(O=em.out, dQ=em.dq, dK=em.dk, dV=em.dv))


@pytest.mark.parametrize("b", BATCH_SIZES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("s_", [1, 2, 63, 64, 65, 127, 128, 129, 1024])
def test_qkvpacked_grid(ext, s_, d, causal, b):
    # qkv-packed entry point over the equal-length cases (test_flash_attn.py:857-932)
    from flash_attention_turing_b200 import flash_attn_qkvpacked_func

    h = 4
    gen = torch.Generator().manual_seed(_seed("qkv", s_, d, causal, b))
    qkv = randn_half(gen, b, s_, 3, h, d).to(DEV)
    dout = randn_half(gen, b, s_, h, d).to(DEV)
    x = qkv.clone().requires_grad_(True)
    out = flash_attn_qkvpacked_func(x, causal=causal)
    (dqkv,) = torch.autograd.grad(out, x, dout)
    q, k, v = (qkv[:, :, i].contiguous() for i in range(3))
    s = d ** -0.5
    o_ref, _ = orc.attention_forward(q, k, v, s, causal)
    rq, rk, rv = orc.attention_backward(q, k, v, dout, s, causal)
    em = emulate_reference_kernel(q, k, v, dout, s, causal)
    _check_all(dict(O=out, dQ=dqkv[:, :, 0], dK=dqkv[:, :, 1], dV=dqkv[:, :, 2]), dict(O=o_ref, dQ=rq, dK=rk, dV=rv),
               dict(O=em.out, dQ=em.dq, dK=em.dk, dV=em.dv))


@pytest.mark.parametrize("num_splits", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("h,hk", [(4, 2), (6, 1)])
@pytest.mark.parametrize("d", [64, 128])
def test_kvcache_randomised_lengths(ext, d, h, hk, causal, num_splits):
    # test_flash_attn.py:1387-1433: batch 3, 7 query tokens, capacity 321, eight draws of the lengths
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    gen = torch.Generator().manual_seed(_seed("kvc", d, h, hk, causal, num_splits))
    b, sq, cap = 3, 7, 321
    q, kc, vc = randn_half(gen, b, sq, h, d).to(DEV), randn_half(gen, b, cap, hk, d).to(DEV), randn_half(gen, b, cap, hk, d).to(DEV)
    for _ in range(8):
        lens = torch.randint(32, cap - 1, (b,), generator=gen, dtype=torch.int32)
        out, lse = flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens.to(DEV), causal=causal, num_splits=num_splits,
                                           return_softmax_lse=True)
        o_ref, lse_ref = orc.attention_forward(q, kc, vc, None, causal, seqlens_k=lens.tolist())
        assert err_stats(out, o_ref)[0] <= 2e-3
        assert err_stats(lse, lse_ref)[0] <= LSE_TOL


@pytest.mark.parametrize("page", [256, 512])
@pytest.mark.parametrize("num_splits", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("h,hk", [(4, 2), (6, 1)])
@pytest.mark.parametrize("d", [64, 128])
def test_kvcache_paged_randomised_lengths(ext, d, h, hk, causal, num_splits, page):
    # test_flash_attn.py:1436-1488: batch 2, 5 query tokens, three pages per sequence, six draws of the lengths
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    gen = torch.Generator().manual_seed(_seed("kvp", d, h, hk, causal, num_splits, page))
    b, sq, per = 2, 5, 3
    cap = page * per
    q = randn_half(gen, b, sq, h, d).to(DEV)
    k_dense, v_dense = randn_half(gen, b, cap, hk, d).to(DEV), randn_half(gen, b, cap, hk, d).to(DEV)
    perm = torch.randperm(b * per, generator=gen)
    table = perm.view(b, per).to(torch.int32)
    k_paged = torch.empty(b * per, page, hk, d, dtype=torch.half, device=DEV)
    v_paged = torch.empty_like(k_paged)
    for i in range(b):
        for j in range(per):
            k_paged[int(table[i, j])] = k_dense[i, j * page:(j + 1) * page]
            v_paged[int(table[i, j])] = v_dense[i, j * page:(j + 1) * page]
    for _ in range(6):
        lens = torch.randint(page // 2, cap - 1, (b,), generator=gen, dtype=torch.int32)
        out, lse = flash_attn_with_kvcache(q, k_paged.clone(), v_paged.clone(), cache_seqlens=lens.to(DEV),
                                           block_table=table.to(DEV), causal=causal, num_splits=num_splits,
                                           return_softmax_lse=True)
        o_ref, lse_ref = orc.attention_forward(q, k_dense, v_dense, None, causal, seqlens_k=lens.tolist())
        assert err_stats(out, o_ref)[0] <= 2e-3
        assert err_stats(lse, lse_ref)[0] <= LSE_TOL


@pytest.mark.parametrize("sq,sk,h,hk,d,causal", [(129, 257, 4, 2, 64, False), (1024, 897, 6, 1, 128, True),
                                                 (64, 2, 6, 3, 128, True), (1, 1024, 2, 1, 64, True)])
def test_oracle_on_device_matches_oracle_on_cpu(sq, sk, h, hk, d, causal):
    # the grid above evaluates the oracle's code on CUDA tensors; this ties that evaluation to the CPU one
    gen = torch.Generator().manual_seed(_seed("dev", sq, sk))
    q, k, v, dout = (randn_half(gen, 2, s, n, d) for s, n in ((sq, h), (sk, hk), (sk, hk), (sq, h)))
    cpu = (*orc.attention_forward(q, k, v, None, causal), *orc.attention_backward(q, k, v, dout, None, causal))
    dev = (*orc.attention_forward(q.to(DEV), k.to(DEV), v.to(DEV), None, causal),
           *orc.attention_backward(q.to(DEV), k.to(DEV), v.to(DEV), dout.to(DEV), None, causal))
    for a, b_ in zip(cpu, dev):
        assert (a - b_.cpu()).abs().max().item() <= 2e-5 * max(1.0, a.abs().max().item())
