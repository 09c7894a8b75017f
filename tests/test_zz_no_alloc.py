"""fa_kvcache_noalloc: the KV-cache step for callers that cannot allocate device memory.

Such callers exist: a serving loop that froze its memory pool at start-up, a plugin running inside
another runtime's stream callback or graph node (cudaMalloc is off limits there), a host language
binding that can launch kernels but has no allocator.  For them the library keeps the split-KV scratch
in an array of its own image (32 MiB per GPU) and this entry point uses it.

The test calls the entry point through the C ABI twice in a row and compares each result with
fa_kvcache() given a caller-owned workspace -- same kernels, so the outputs must agree to the tolerance the
other KV-cache tests use (they are in fact bit-identical) -- and with the CPU oracle.  The second call reuses the scratch the first
one left behind, on different inputs, which proves that stale contents do no harm.  It also checks that
a request beyond the built-in limit is refused with an error code instead of being launched.

This file sorts last on purpose, so that a run that stops at the first failure has already run every
other test; it passes on its own in a fresh process as well.
"""
import ctypes

import pytest
import torch

from helpers import randn_half

pytestmark = pytest.mark.gpu
DEV = "cuda"
O_TOL = 2e-3
LSE_TOL = 1e-3


def _case(seed, b, h, hk, d, page, per, lens, splits):
    from flash_attention_turing_b200 import capi

    gen = torch.Generator().manual_seed(seed)
    n_pages = b * per + 1
    kc, vc = randn_half(gen, n_pages, page, hk, d).to(DEV), randn_half(gen, n_pages, page, hk, d).to(DEV)
    table = torch.randperm(n_pages, generator=gen)[: b * per].to(torch.int32).view(b, per).contiguous().to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = randn_half(gen, b, 1, h, d).to(DEV)
    kn, vn = randn_half(gen, b, 1, hk, d).to(DEV), randn_half(gen, b, 1, hk, d).to(DEV)

    def params(k_cache, v_cache, out, lse):
        return capi.kvcache_params(q, k_cache, v_cache, kn, vn, out, lse, lens_d, table, d ** -0.5, True, splits)

    return params, kc, vc, q, kn, vn, table


def _run_both(lib, stream, seed, lens, splits):
    from flash_attention_turing_b200 import capi

    b, h, hk, d, page, per = len(lens), 8, 2, 128, 256, 8
    params, kc, vc, q, kn, vn, p2_table = _case(seed, b, h, hk, d, page, per, lens, splits)
    # existing entry point, caller-owned workspace
    kc1, vc1 = kc.clone(), vc.clone()
    o1, l1 = torch.empty_like(q), torch.empty(b, h, 1, dtype=torch.float32, device=DEV)
    p1 = params(kc1, vc1, o1, l1)
    need = lib.fa_kvcache_workspace_bytes(ctypes.byref(p1))
    assert need > 0, "the case must use split scratch"
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    p1.workspace, p1.workspace_bytes = ws.data_ptr(), need
    capi.check(lib.fa_kvcache(ctypes.byref(p1), stream))
    # entry point under test: no workspace passed at all
    kc2, vc2 = kc.clone(), vc.clone()
    o2, l2 = torch.empty_like(q), torch.empty(b, h, 1, dtype=torch.float32, device=DEV)
    p2 = params(kc2, vc2, o2, l2)
    capi.check(lib.fa_kvcache_noalloc(ctypes.byref(p2), stream))
    torch.cuda.synchronize()
    assert not torch.isnan(o2).any()
    assert (o2.float() - o1.float()).abs().max().item() <= O_TOL
    assert (l2 - l1).abs().max().item() <= LSE_TOL
    assert torch.equal(kc2, kc1) and torch.equal(vc2, vc1)  # the in-place append is the same too
    # ... and against the CPU oracle, not only against the sibling entry point
    from oracle import attention_oracle as orc

    table = p2_table.cpu()
    lens_t = torch.tensor(lens, dtype=torch.int32)
    o_ref, lse_ref = orc.kvcache_forward(q.cpu(), kc.cpu(), vc.cpu(), kn.cpu(), vn.cpu(), lens_t, None, table,
                                         d ** -0.5, True)
    assert (o2.float().cpu() - o_ref).abs().max().item() <= O_TOL
    assert (l2.cpu() - lse_ref).abs().max().item() <= LSE_TOL


def test_noalloc_matches_fa_kvcache_on_two_calls_in_a_row():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _run_both(lib, stream, seed=101, lens=[1900, 37, 1024], splits=4)
    # second call: other inputs, other split count, same built-in scratch with the first call's leftovers
    _run_both(lib, stream, seed=202, lens=[5, 2047, 700, 1300], splits=7)
    assert lib.fa_device_status(1) == 0


def test_noalloc_rejects_requests_beyond_the_builtin_scratch():
    from flash_attention_turing_b200 import capi

    lib = capi.lib()
    p = capi.FaKvcacheParams()
    # 64 splits x (256 x 32 x 1 rows) x 128 x 4 B = 268 MB of partials: far beyond 32 MiB
    p.b, p.seqlen_q, p.h, p.h_k, p.d, p.cache_batch, p.seqlen_cache, p.num_splits = 256, 1, 32, 8, 128, 256, 4096, 64
    assert lib.fa_kvcache_workspace_bytes(ctypes.byref(p)) > 32 * 1024 * 1024
    rc = lib.fa_kvcache_noalloc(ctypes.byref(p), None)
    assert rc == -3
    assert b"built-in" in lib.fa_last_error()
