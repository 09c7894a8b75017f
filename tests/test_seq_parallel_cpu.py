"""World-size-2 (and 4) gloo tests of the sequence-sharded forward's and backward's exchange logic on CPU ranks.

The kernels are injected: the CPU oracle stands in for the forward kernel and for the combine kernel,
so what is tested here is the sharding arithmetic (causal offsets per shard), the all-to-all layout and
the merge -- not any CPU execution path of the product (there is none)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as orc


def _oracle_fwd(q, k, v, scale, causal):
    out, lse = orc.attention_forward(q, k, v, scale, causal)
    # a row without a visible key: the kernels return LSE = 0 there; partial_attention never asks for such rows
    return out.to(q.dtype), lse


def _oracle_combine(o_accum, lse_accum, b, sq, h):
    out, lse = orc.combine(o_accum, lse_accum)
    d = out.shape[-1]
    return out.view(b, h, sq, d).permute(0, 2, 1, 3).contiguous(), lse.view(b, h, sq)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_attention_turing_b200 import seq_parallel as sp

        torch.manual_seed(5)  # same data on every rank
        b, s, h, hk, d = 2, 64, 4, 2, 64
        q = torch.randn(b, s, h, d)
        k = torch.randn(b, s, hk, d)
        v = torch.randn(b, s, hk, d)
        shard = s // world
        ks, vs = k[:, rank * shard:(rank + 1) * shard], v[:, rank * shard:(rank + 1) * shard]
        out, lse = sp.sequence_parallel_forward(q, ks, vs, None, causal, gather_output=True,
                                                fwd=_oracle_fwd, combine=_oracle_combine)
        ref_out, ref_lse = orc.attention_forward(q, k, v, None, causal)
        err_o = (out - ref_out).abs().max().item()
        err_l = (lse - ref_lse).abs().max().item()
        # slice-only result too
        out_s, _ = sp.sequence_parallel_forward(q, ks, vs, None, causal, fwd=_oracle_fwd, combine=_oracle_combine)
        sl = s // world
        err_s = (out_s - ref_out[:, rank * sl:(rank + 1) * sl]).abs().max().item()
        results[rank] = (err_o, err_l, err_s)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_sequence_parallel_forward_matches_single_process(world, causal):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), causal, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        err_o, err_l, err_s = results[rank]
        assert err_o < 1e-5 and err_l < 1e-5 and err_s < 1e-5, (rank, err_o, err_l, err_s)


def test_partial_attention_rows_before_the_shard_are_neutral():
    from flash_attention_turing_b200 import seq_parallel as sp

    torch.manual_seed(0)
    q, k, v = torch.randn(1, 16, 2, 64), torch.randn(1, 4, 2, 64), torch.randn(1, 4, 2, 64)
    out, lse = sp.partial_attention(q, k, v, key_offset=8, softmax_scale=0.125, causal=True, fwd=_oracle_fwd)
    assert torch.isinf(lse[:, :, :8]).all() and (lse[:, :, :8] < 0).all()
    assert out[:, :8].abs().max().item() == 0
    assert torch.isfinite(lse[:, :, 8:]).all()


# ------------------------------------------------------------------------------------------------
# backward: shard-local dK/dV, dQ shares summed across ranks
# ------------------------------------------------------------------------------------------------
def _oracle_bwd(q, k, v, out, lse, dout, scale, causal):
    return orc.attention_backward_given_lse(q, k, v, out, lse, dout, scale, causal)


def _oracle_sum(shares):
    return shares.float().sum(0)


def _bwd_worker(rank, world, port, causal, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_attention_turing_b200 import seq_parallel as sp

        torch.manual_seed(9)  # same data on every rank
        b, s, h, hk, d = 2, 64, 4, 2, 64
        q, dout = torch.randn(b, s, h, d), torch.randn(b, s, h, d)
        k, v = torch.randn(b, s, hk, d), torch.randn(b, s, hk, d)
        shard = s // world
        ks, vs = k[:, rank * shard:(rank + 1) * shard], v[:, rank * shard:(rank + 1) * shard]
        out, lse = sp.sequence_parallel_forward(q, ks, vs, None, causal, gather_output=True,
                                                fwd=_oracle_fwd, combine=_oracle_combine)
        dq, dk, dv = sp.sequence_parallel_backward(q, ks, vs, out, lse, dout, None, causal,
                                                   bwd=_oracle_bwd, sum_parts=_oracle_sum)
        rq, rk, rv = orc.attention_backward(q, k, v, dout, None, causal)
        sl = s // world
        results[rank] = ((dq - rq[:, rank * sl:(rank + 1) * sl]).abs().max().item(),
                         (dk - rk[:, rank * shard:(rank + 1) * shard]).abs().max().item(),
                         (dv - rv[:, rank * shard:(rank + 1) * shard]).abs().max().item())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_sequence_parallel_backward_matches_single_process(world, causal):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_bwd_worker, args=(world, _free_port(), causal, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        assert max(results[rank]) < 2e-5, (rank, results[rank])


def test_backward_from_saved_statistics_equals_recomputed_backward():
    torch.manual_seed(3)
    q, dout = torch.randn(1, 24, 4, 64), torch.randn(1, 24, 4, 64)
    k, v = torch.randn(1, 40, 2, 64), torch.randn(1, 40, 2, 64)
    for causal in (False, True):
        out, lse = orc.attention_forward(q, k, v, None, causal)
        got = orc.attention_backward_given_lse(q, k, v, out, lse, dout, None, causal)
        want = orc.attention_backward(q, k, v, dout, None, causal)
        for g, w in zip(got, want):
            assert (g - w).abs().max().item() < 1e-5


def test_partial_backward_rows_before_the_shard_get_no_gradient():
    from flash_attention_turing_b200 import seq_parallel as sp

    torch.manual_seed(1)
    q, dout = torch.randn(1, 16, 2, 64), torch.randn(1, 16, 2, 64)
    k, v = torch.randn(1, 16, 2, 64), torch.randn(1, 16, 2, 64)
    out, lse = orc.attention_forward(q, k, v, 0.125, True)
    dq, dk, dv = sp.partial_backward(q, k[:, 8:12], v[:, 8:12], out, lse, dout, key_offset=8, softmax_scale=0.125,
                                     causal=True, bwd=_oracle_bwd)
    assert dq[:, :8].abs().max().item() == 0
    assert dq[:, 8:].abs().max().item() > 0
    rq, rk, rv = orc.attention_backward(q, k, v, dout, 0.125, True)
    assert (dk - rk[:, 8:12]).abs().max().item() < 1e-5 and (dv - rv[:, 8:12]).abs().max().item() < 1e-5


# ------------------------------------------------------------------------------------------------
# zig-zag layout: two chunks per rank, merged locally before the exchange
# ------------------------------------------------------------------------------------------------
def _oracle_merge2(o_parts, lse_parts):
    b, s, h, d = o_parts[0].shape
    o_acc = torch.stack([o.float().permute(0, 2, 1, 3).reshape(b * h * s, d) for o in o_parts])
    l_acc = torch.stack([l.reshape(b * h * s) for l in lse_parts])
    out, lse = orc.combine(o_acc, l_acc)
    return out.view(b, h, s, d).permute(0, 2, 1, 3).contiguous(), lse.view(b, h, s)


def _oracle_add2(parts):
    return parts[0].float() + parts[1].float()


def _zigzag_worker(rank, world, port, causal, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_attention_turing_b200 import seq_parallel as sp

        torch.manual_seed(13)
        b, s, h, hk, d = 1, 64, 4, 2, 64
        q, dout = torch.randn(b, s, h, d), torch.randn(b, s, h, d)
        k, v = torch.randn(b, s, hk, d), torch.randn(b, s, hk, d)
        ks, vs = sp.shard_kv(k, rank, world, "zigzag"), sp.shard_kv(v, rank, world, "zigzag")
        out, lse = sp.sequence_parallel_forward(q, ks, vs, None, causal, gather_output=True, fwd=_oracle_fwd,
                                                combine=_oracle_combine, layout="zigzag", merge2=_oracle_merge2)
        dq, dk, dv = sp.sequence_parallel_backward(q, ks, vs, out, lse, dout, None, causal, bwd=_oracle_bwd,
                                                   sum_parts=_oracle_sum, layout="zigzag", add2=_oracle_add2)
        ref_out, ref_lse = orc.attention_forward(q, k, v, None, causal)
        rq, rk, rv = orc.attention_backward(q, k, v, dout, None, causal)
        sl = s // world
        results[rank] = ((out - ref_out).abs().max().item(), (lse - ref_lse).abs().max().item(),
                         (dq - rq[:, rank * sl:(rank + 1) * sl]).abs().max().item(),
                         (dk - sp.shard_kv(rk, rank, world, "zigzag")).abs().max().item(),
                         (dv - sp.shard_kv(rv, rank, world, "zigzag")).abs().max().item())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_zigzag_layout_matches_single_process(world, causal):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_zigzag_worker, args=(world, _free_port(), causal, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        assert max(results[rank]) < 2e-5, (rank, results[rank])


def test_shard_chunks():
    from flash_attention_turing_b200 import seq_parallel as sp

    assert sp.shard_chunks(1, 4, 64) == [(16, 32)]
    assert sp.shard_chunks(1, 4, 64, "zigzag") == [(8, 16), (48, 56)]
    covered = sorted(c for r in range(4) for c in sp.shard_chunks(r, 4, 64, "zigzag"))
    assert covered == [(8 * i, 8 * i + 8) for i in range(8)]
    with pytest.raises(ValueError):
        sp.shard_chunks(0, 4, 36, "zigzag")
    with pytest.raises(ValueError):
        sp.shard_chunks(0, 4, 64, "striped")


def test_owned_rows_balance_the_merge_under_a_causal_mask():
    """Row ownership of the peer-read paths: one contiguous slice per rank, or the rows of the rank's two zig-zag
    chunks.  The number of (row chunk, K/V chunk) pairs a rank has to fetch and merge under a causal mask -- a row
    chunk sees the K/V chunks up to its own -- is the same on every rank only with the zig-zag rows."""
    import torch

    from flash_attention_turing_b200 import seq_parallel as sp

    world, s = 8, 1024
    assert sp.owned_rows(3, world, s) == [(384, 512)]
    assert sp.owned_rows(3, world, s, "zigzag") == [(192, 256), (768, 832)]
    c = s // (2 * world)

    def pairs(rows):  # (row chunk, visible K/V chunk) pairs: row chunk i sees the K/V chunks 0 .. i
        return sum(i + 1 for b, e in rows for i in range(b // c, e // c))

    contiguous = [pairs(sp.owned_rows(r, world, s)) for r in range(world)]
    zigzag = [pairs(sp.owned_rows(r, world, s, "zigzag")) for r in range(world)]
    assert max(contiguous) == 31 and min(contiguous) == 3
    assert set(zigzag) == {17}
    x = torch.arange(s).view(1, s, 1, 1)
    got = sp.gather_owned_rows(x, 3, world, "zigzag").flatten().tolist()
    assert got == list(range(192, 256)) + list(range(768, 832))
    every = sorted(v for r in range(world) for v in sp.gather_owned_rows(x, r, world, "zigzag").flatten().tolist())
    assert every == list(range(s))
