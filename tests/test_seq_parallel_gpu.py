"""Sequence-sharded forward and backward on two GPUs over NCCL, checked against the single-GPU kernels and
the CPU oracle.  Skipped on a box with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _require_peer_path(errs, tol):
    """The fused peer-read path ran on every rank and agrees with the all-to-all path; when the peers' memory
    cannot be mapped on this machine the test says so as a skip instead of passing silently."""
    if any(e < 0 for e in errs):
        pytest.skip("symmetric memory unavailable: the fused peer-read path was not exercised")
    assert max(errs) <= tol, errs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, d, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flash_attention_turing_b200 import _ext, seq_parallel as sp
        from oracle import attention_oracle as orc

        ext = _ext.load()
        gen = torch.Generator().manual_seed(11)  # same data on every rank
        b, s, h, hk = 1, 1024, 4, 2
        q = torch.randn(b, s, h, d, generator=gen).half()
        k = torch.randn(b, s, hk, d, generator=gen).half()
        v = torch.randn(b, s, hk, d, generator=gen).half()
        shard = s // world
        qd = q.to(dev)
        ks = k[:, rank * shard:(rank + 1) * shard].contiguous().to(dev)
        vs = v[:, rank * shard:(rank + 1) * shard].contiguous().to(dev)
        out, lse = sp.sequence_parallel_forward(qd, ks, vs, None, causal, gather_output=True)
        torch.cuda.synchronize()
        # fused exchange + merge over peer memory must give the same slice as the all-to-all path; whether
        # symmetric memory can be used is agreed on by all ranks on the host BEFORE anyone enters a device-side
        # barrier, so that no rank waits for a peer that gave up
        p2p_err = -1.0
        if sp.peer_memory_available_for(qd):
            out_p, lse_p = sp.sequence_parallel_forward_p2p(qd, ks, vs, None, causal)
            torch.cuda.synchronize()
            sl = s // world
            p2p_err = max((out_p.float() - out[:, rank * sl:(rank + 1) * sl].float()).abs().max().item(),
                          (lse_p - lse[:, :, rank * sl:(rank + 1) * sl]).abs().max().item())
        ref_out, ref_lse = orc.attention_forward(q, k, v, None, causal)
        one_out, _ = ext.fwd(qd, k.to(dev), v.to(dev), d ** -0.5, causal)
        results[rank] = ((out.float().cpu() - ref_out).abs().max().item(),
                         (lse.cpu() - ref_lse).abs().max().item(),
                         (out.float() - one_out.float()).abs().max().item(),
                         int(ext.device_status(True)), p2p_err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_two_gpu_sequence_parallel_forward(causal, d):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), causal, d, results), nprocs=world, join=True)
    for rank in range(world):
        err_o, err_l, err_one, status, p2p_err = results[rank]
        assert status == 0
        assert err_o <= 3e-3, (rank, err_o)       # fp16 partials merged: two fp16 roundings
        assert err_l <= 1e-3, (rank, err_l)
        assert err_one <= 3e-3, (rank, err_one)
    _require_peer_path([results[r][4] for r in range(world)], 1e-3)


def _bwd_worker(rank, world, port, causal, d, results, layout="contiguous"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flash_attention_turing_b200 import _ext, seq_parallel as sp
        from oracle import attention_oracle as orc

        ext = _ext.load()
        gen = torch.Generator().manual_seed(17)  # same data on every rank
        b, s, h, hk = 1, 1024, 4, 2
        q = torch.randn(b, s, h, d, generator=gen).half()
        k = torch.randn(b, s, hk, d, generator=gen).half()
        v = torch.randn(b, s, hk, d, generator=gen).half()
        dout = torch.randn(b, s, h, d, generator=gen).half()
        sl = s // world
        qd, dod = q.to(dev), dout.to(dev)
        ks, vs = sp.shard_kv(k, rank, world, layout).to(dev), sp.shard_kv(v, rank, world, layout).to(dev)
        out, lse = sp.sequence_parallel_forward(qd, ks, vs, None, causal, gather_output=True, layout=layout)
        dq, dk, dv = sp.sequence_parallel_backward(qd, ks, vs, out, lse, dod, None, causal, layout=layout)
        torch.cuda.synchronize()
        p2p_err = -1.0
        if sp.peer_memory_available_for(qd, layout):
            out_p, lse_p = sp.sequence_parallel_forward_p2p(qd, ks, vs, None, causal, layout=layout)
            fwd_p2p = max((out_p.float() - out[:, rank * sl:(rank + 1) * sl].float()).abs().max().item(),
                          (lse_p - lse[:, :, rank * sl:(rank + 1) * sl]).abs().max().item())
            assert fwd_p2p <= 2e-3, fwd_p2p  # zig-zag: parts are merged in one step instead of two
            dq_p, dk_p, dv_p = sp.sequence_parallel_backward_p2p(qd, ks, vs, out, lse, dod, None, causal, layout=layout)
            torch.cuda.synchronize()
            p2p_err = max((dq_p.float() - dq.float()).abs().max().item(), (dk_p.float() - dk.float()).abs().max().item(),
                          (dv_p.float() - dv.float()).abs().max().item())
        rq, rk, rv = orc.attention_backward(q, k, v, dout, None, causal)
        ref_out, _ = orc.attention_forward(q, k, v, None, causal)
        errs = ((dq.float().cpu() - rq[:, rank * sl:(rank + 1) * sl]).abs().max().item(),
                (dk.float().cpu() - sp.shard_kv(rk, rank, world, layout)).abs().max().item(),
                (dv.float().cpu() - sp.shard_kv(rv, rank, world, layout)).abs().max().item(),
                (out.float().cpu() - ref_out).abs().max().item())
        scale = max(rq.abs().max().item(), rk.abs().max().item(), rv.abs().max().item())
        results[rank] = (errs, scale, int(ext.device_status(True)), p2p_err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_two_gpu_sequence_parallel_backward(causal, d):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_bwd_worker, args=(world, _free_port(), causal, d, results), nprocs=world, join=True)
    for rank in range(world):
        errs, scale, status, p2p_err = results[rank]
        assert status == 0
        # fp16 gradients, the dQ shares rounded to fp16 before they are summed
        assert max(errs) <= 4e-3 + 2.0 ** -9 * scale, (rank, errs, scale)
    _require_peer_path([results[r][3] for r in range(world)], 1e-6)  # same kernels, same order of additions


@pytest.mark.parametrize("d", [64, 128])
def test_two_gpu_zigzag_layout_forward_and_backward(d):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_bwd_worker, args=(world, _free_port(), True, d, results, "zigzag"), nprocs=world, join=True)
    for rank in range(world):
        errs, scale, status, p2p_err = results[rank]
        assert status == 0
        # one more fp16 rounding than the contiguous layout: the two chunks' results are merged locally
        assert max(errs) <= 5e-3 + 2.0 ** -9 * scale, (rank, errs, scale)
    # the peer-read path sums the four chunk shares in one step, the all-to-all path adds each rank's two
    # first (one more fp16 rounding): they agree to an fp16 ulp, not bit for bit
    _require_peer_path([results[r][3] for r in range(world)], 1e-3)
