"""Calls libfa_b200.so exactly as a non-Python host would -- ctypes, raw device pointers, explicit
strides and stream -- and checks the results against the CPU oracle."""
import ctypes

import pytest
import torch

from helpers import LSE_TOL, MAX_ABS_TOL, err_stats, randn_half
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ptr(x):
    return ctypes.c_void_p(x.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_fa_fwd_and_fa_bwd_raw():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    b, sq, sk, h, hk, d = 2, 200, 333, 4, 2, 128
    gen = torch.Generator().manual_seed(9)
    q, k, v, dout = (randn_half(gen, *s) for s in ((b, sq, h, d), (b, sk, hk, d), (b, sk, hk, d), (b, sq, h, d)))
    qd, kd, vd, dd = (x.to(DEV) for x in (q, k, v, dout))
    o = torch.empty_like(qd)
    lse = torch.empty(b, h, sq, dtype=torch.float32, device=DEV)
    p = capi.FaFwdParams()
    p.q, p.k, p.v, p.o, p.lse = _ptr(qd), _ptr(kd), _ptr(vd), _ptr(o), _ptr(lse)
    for name, x in (("q", qd), ("k", kd), ("v", vd), ("o", o)):
        setattr(p, f"{name}_batch_stride", x.stride(0))
        setattr(p, f"{name}_row_stride", x.stride(1))
        setattr(p, f"{name}_head_stride", x.stride(2))
    p.lse_row_stride = sq
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d, p.k_batch = b, sq, sk, h, hk, d, b
    p.softmax_scale, p.is_causal = d ** -0.5, 1
    capi.check(lib.fa_fwd(ctypes.byref(p), _stream()))
    o_ref, lse_ref = orc.attention_forward(q, k, v, None, True)
    assert err_stats(o, o_ref)[0] <= MAX_ABS_TOL and err_stats(lse, lse_ref)[0] <= LSE_TOL

    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    bp = capi.FaBwdParams()
    bp.q, bp.k, bp.v, bp.o, bp.dout, bp.lse = _ptr(qd), _ptr(kd), _ptr(vd), _ptr(o), _ptr(dd), _ptr(lse)
    bp.dq, bp.dk, bp.dv = _ptr(dq), _ptr(dk), _ptr(dv)
    for name, x in (("q", qd), ("k", kd), ("v", vd), ("o", o), ("do", dd), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(bp, f"{name}_batch_stride", x.stride(0))
        setattr(bp, f"{name}_row_stride", x.stride(1))
        setattr(bp, f"{name}_head_stride", x.stride(2))
    bp.lse_row_stride = sq
    bp.b, bp.seqlen_q, bp.seqlen_k, bp.h, bp.h_k, bp.d = b, sq, sk, h, hk, d
    bp.softmax_scale, bp.is_causal = d ** -0.5, 1
    need = lib.fa_bwd_workspace_bytes(ctypes.byref(bp))
    # too small a workspace is an error code, not a fault
    small = torch.empty(16, dtype=torch.uint8, device=DEV)
    bp.workspace, bp.workspace_bytes = _ptr(small), 16
    assert lib.fa_bwd(ctypes.byref(bp), _stream()) == -3
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    bp.workspace, bp.workspace_bytes = _ptr(ws), need
    capi.check(lib.fa_bwd(ctypes.byref(bp), _stream()))
    rq, rk, rv = orc.attention_backward(q, k, v, dout, None, True)
    for got, want in ((dq, rq), (dk, rk), (dv, rv)):
        assert err_stats(got, want)[0] <= MAX_ABS_TOL
    assert lib.fa_device_status(1) == 0


def test_fa_combine_raw():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    n, b, h, sq, d = 5, 2, 3, 4, 128
    rows = b * h * sq
    gen = torch.Generator().manual_seed(3)
    o_acc = torch.randn(n, rows, d, generator=gen)
    l_acc = torch.randn(n, rows, generator=gen) * 3
    l_acc[1, 5] = float("-inf")          # an empty split for one row
    l_acc[:, 7] = float("-inf")          # a row whose every split is empty
    o_acc[:, 7] = float("nan")           # ... whose partials must not be read into the result
    want_o, want_l = orc.combine(torch.nan_to_num(o_acc), l_acc)
    oa, la = o_acc.to(DEV), l_acc.to(DEV)
    out = torch.empty(b, sq, h, d, dtype=torch.half, device=DEV)
    lse = torch.empty(b, h, sq, dtype=torch.float32, device=DEV)
    p = capi.FaCombineParams()
    p.o_accum, p.lse_accum, p.o, p.lse = _ptr(oa), _ptr(la), _ptr(out), _ptr(lse)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
    p.num_splits, p.b, p.h, p.seqlen_q, p.d = n, b, h, sq, d
    capi.check(lib.fa_combine(ctypes.byref(p), _stream()))
    got = out.float().cpu().permute(0, 2, 1, 3).reshape(rows, d)  # (b, h, sq) row order
    assert err_stats(got, want_o)[0] <= 4e-3
    assert err_stats(lse.view(-1), want_l)[0] <= 1e-5
    assert out.float().cpu().permute(0, 2, 1, 3).reshape(rows, d)[7].abs().max().item() == 0


@pytest.mark.parametrize("n,b,s,h,d,row_begin,rows", [(2, 2, 10, 3, 64, 4, 5), (8, 1, 33, 2, 128, 0, 33),
                                                    (5, 2, 16, 4, 128, 15, 1), (16, 1, 9, 1, 64, 2, 6)])
def test_fa_combine_gather_raw_on_one_gpu(n, b, s, h, d, row_begin, rows):
    """The merge of per-rank partials, here with all parts in this GPU's own memory (the kernel does not care
    whose memory a part pointer names): 2 to 16 parts in the forward's layout, a row slice, empty parts
    (LSE = -inf) whose O holds NaN and must not be read into the result, and one row that every part left
    empty.  Expected values: the oracle's combine on the same slice."""
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    gen = torch.Generator().manual_seed(100 + n)
    o_parts = [torch.randn(b, s, h, d, generator=gen).half() for _ in range(n)]
    l_parts = [torch.randn(b, h, s, generator=gen) * 3 for _ in range(n)]
    l_parts[0][:, :, row_begin] = float("-inf")      # part 0 saw no key for the first row of the slice
    o_parts[0][:, row_begin] = float("nan")
    dead_row = row_begin + rows - 1
    for r in range(n):                               # a row nobody saw a key for
        l_parts[r][0, 0, dead_row] = float("-inf")
        o_parts[r][0, dead_row, 0] = float("nan")
    sl = slice(row_begin, row_begin + rows)
    o_acc = torch.stack([torch.nan_to_num(x[:, sl].float()).permute(0, 2, 1, 3).reshape(-1, d) for x in o_parts])
    l_acc = torch.stack([x[:, :, sl].reshape(-1) for x in l_parts])
    want_o, want_l = orc.combine(o_acc, l_acc)                          # rows ordered (b, h, row)
    od, ld = [x.to(DEV) for x in o_parts], [x.to(DEV) for x in l_parts]
    out = torch.full((b, rows, h, d), float("nan"), dtype=torch.half, device=DEV)
    lse = torch.full((b, h, rows), float("nan"), dtype=torch.float32, device=DEV)
    p = capi.FaCombineGatherParams()
    for i in range(n):
        p.o_part[i], p.lse_part[i] = od[i].data_ptr(), ld[i].data_ptr()
    p.o, p.lse = out.data_ptr(), lse.data_ptr()
    p.num_parts, p.b, p.h, p.seqlen_q, p.d, p.row_begin, p.rows = n, b, h, s, d, row_begin, rows
    capi.check(lib.fa_combine_gather(ctypes.byref(p), _stream()))
    torch.cuda.synchronize()
    got = out.float().cpu().permute(0, 2, 1, 3).reshape(-1, d)
    assert not torch.isnan(got).any()
    assert err_stats(got, want_o)[0] <= 2.0 ** -10 * max(1.0, want_o.abs().max().item())  # one fp16 rounding
    assert err_stats(lse.view(-1), want_l)[0] <= 1e-5
    assert out[0, rows - 1, 0].abs().max().item() == 0 and lse[0, 0, rows - 1].item() == 0
    p.num_parts = 17
    assert lib.fa_combine_gather(ctypes.byref(p), _stream()) != 0
    assert lib.fa_device_status(1) == 0


def test_fa_sum_gather_raw():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    for n, b, s, h, d, row_begin, rows in ((3, 2, 10, 3, 64, 4, 5), (16, 1, 7, 2, 128, 0, 7), (1, 2, 4, 1, 64, 3, 1)):
        gen = torch.Generator().manual_seed(n)
        parts = [torch.randn(b, s, h, d, generator=gen).half() for _ in range(n)]
        want = sum(x[:, row_begin:row_begin + rows].float() for x in parts)
        dev_parts = [x.to(DEV) for x in parts]
        out = torch.empty(b, rows, h, d, dtype=torch.half, device=DEV)
        p = capi.FaSumGatherParams()
        for i, x in enumerate(dev_parts):
            p.part[i] = x.data_ptr()
        p.out = out.data_ptr()
        p.num_parts, p.b, p.h, p.seqlen_q, p.d, p.row_begin, p.rows = n, b, h, s, d, row_begin, rows
        capi.check(lib.fa_sum_gather(ctypes.byref(p), _stream()))
        torch.cuda.synchronize()
        # fp32 sum rounded once to fp16
        assert torch.equal(out.cpu(), want.half())
    p.num_parts = 17
    assert lib.fa_sum_gather(ctypes.byref(p), _stream()) != 0
    assert b"num_parts" in lib.fa_last_error()


def test_fa_kvcache_raw_paged():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    b, h, hk, d, page, per = 3, 8, 2, 128, 256, 6
    gen = torch.Generator().manual_seed(12)
    n_pages = b * per + 2
    kc, vc = randn_half(gen, n_pages, page, hk, d), randn_half(gen, n_pages, page, hk, d)
    table = torch.randperm(n_pages, generator=gen)[: b * per].to(torch.int32).view(b, per).contiguous()
    lens = torch.tensor([17, 1500, 1279], dtype=torch.int32)
    q, kn, vn = randn_half(gen, b, 1, h, d), randn_half(gen, b, 1, hk, d), randn_half(gen, b, 1, hk, d)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    o_ref, lse_ref = orc.kvcache_forward(q, kc_ref, vc_ref, kn, vn, lens, None, table, None, True)
    qd, kcd, vcd, knd, vnd, ld, td = (x.to(DEV) for x in (q, kc, vc, kn, vn, lens, table))
    out = torch.empty_like(qd)
    lse = torch.empty(b, h, 1, dtype=torch.float32, device=DEV)
    p = capi.FaKvcacheParams()
    p.q, p.k_cache, p.v_cache, p.k_new, p.v_new, p.o, p.lse = (_ptr(x) for x in (qd, kcd, vcd, knd, vnd, out, lse))
    for name, x in (("q", qd), ("kc", kcd), ("vc", vcd), ("kn", knd), ("vn", vnd), ("o", out)):
        setattr(p, f"{name}_batch_stride", x.stride(0))
        setattr(p, f"{name}_row_stride", x.stride(1))
        setattr(p, f"{name}_head_stride", x.stride(2))
    p.b, p.seqlen_q, p.seqlen_new, p.h, p.h_k, p.d = b, 1, 1, h, hk, d
    p.cache_batch, p.seqlen_cache = n_pages, page
    p.softmax_scale, p.is_causal = d ** -0.5, 1
    p.cache_seqlens, p.block_table = _ptr(ld), _ptr(td)
    p.block_table_batch_stride, p.max_blocks_per_seq = per, per
    for splits in (1, 4, 0):
        p.num_splits = splits
        need = lib.fa_kvcache_workspace_bytes(ctypes.byref(p))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
        p.workspace, p.workspace_bytes = _ptr(ws), need
        capi.check(lib.fa_kvcache(ctypes.byref(p), _stream()))
        assert err_stats(out, o_ref)[0] <= 2e-3 and err_stats(lse, lse_ref)[0] <= LSE_TOL
    assert torch.equal(kcd.cpu(), kc_ref) and torch.equal(vcd.cpu(), vc_ref)
    assert lib.fa_device_status(1) == 0


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """Failure detection without a failure: fa_selftest_wait_timeout() makes one bounded wait run out after
    2 ms (a barrier nobody arrives on, the kernels' own wait routine with a short limit).  The kernel returns by
    itself, bit 0 of the status word is set with the self-test's tag in bits 8-15, a launch issued while the bit
    is set does no work, and after the word is cleared everything works as before."""
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    assert lib.fa_device_status(1) == 0
    capi.check(lib.fa_selftest_wait_timeout(2000, _stream()))
    status = lib.fa_device_status(0)
    assert status & 1 and (status >> 8) & 0xff == 0x7f, hex(status)
    # sticky: a forward launched now leaves its output untouched and the host call still reports success
    b, s, h, d = 1, 128, 1, 64
    gen = torch.Generator().manual_seed(2)
    q, k, v = (randn_half(gen, b, s, h, d).to(DEV) for _ in range(3))
    o = torch.full_like(q, 7.0)
    lse = torch.empty(b, h, s, dtype=torch.float32, device=DEV)
    fp = capi.fwd_params(q, k, v, o, lse, d ** -0.5, False)
    capi.check(lib.fa_fwd(ctypes.byref(fp), _stream()))
    torch.cuda.synchronize()
    assert bool((o == 7.0).all())
    # ... and so does a backward (its kernels take the decision at their first CTA-wide synchronisation)
    dq, dk, dv = (torch.full_like(q, 7.0) for _ in range(3))
    bp = capi.bwd_params(q, k, v, o, torch.ones_like(q), lse, dq, dk, dv, None, d ** -0.5, False)
    need = lib.fa_bwd_workspace_bytes(ctypes.byref(bp))
    ws = torch.empty(max(int(need), 1), dtype=torch.uint8, device=DEV)
    bp.workspace, bp.workspace_bytes = ws.data_ptr(), need
    capi.check(lib.fa_bwd(ctypes.byref(bp), _stream()))
    torch.cuda.synchronize()
    assert all(bool((x == 7.0).all()) for x in (dq, dk, dv))
    assert lib.fa_device_status(1) & 1  # read and clear
    assert lib.fa_device_status(0) == 0
    capi.check(lib.fa_fwd(ctypes.byref(fp), _stream()))
    o_ref, _ = orc.attention_forward(q.cpu(), k.cpu(), v.cpu(), None, False)
    assert err_stats(o, o_ref)[0] <= 2e-3
    assert lib.fa_device_status(1) == 0
