"""GPU parity of flash_attn_with_kvcache (append + attend + split merge) against the CPU oracle.
Mirrors the functional groups of the reference's KV-cache tests (test_flash_attn.py:1104-1964 of
Cy-47/flash-attention-turing): read, append with cache-content check, explicit splits, paged read and
append, shuffled block tables, page sizes 256/512/768/1024, cache_batch_idx, scale, LSE, int lengths,
MHA, and query chunks of several tokens (decode kernel up to 16 rows per KV head, tiled kernel above)."""
import pytest
import torch

from helpers import LSE_TOL, err_stats, load_golden, randn_half, t
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
O_TOL = 2e-3  # fp16 output rounding of O(1) values; the reference's own bound is atol = rtol = 1e-2


def _run(b, sq, h, hk, d, cap, lens, s_new, paged=False, page=256, splits=0, causal=True, batch_idx=False,
         scale=None, seed=7, poison_tail=False):
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    gen = torch.Generator().manual_seed(seed)
    q = randn_half(gen, b, sq, h, d)
    kn = randn_half(gen, b, s_new, hk, d) if s_new else None
    vn = randn_half(gen, b, s_new, hk, d) if s_new else None
    lens_t = torch.tensor(lens, dtype=torch.int32)
    table = idx = None
    if paged:
        per = (cap + page - 1) // page
        n_pages = b * per + 3
        kc, vc = randn_half(gen, n_pages, page, hk, d), randn_half(gen, n_pages, page, hk, d)
        table = torch.randperm(n_pages, generator=gen)[: b * per].to(torch.int32).view(b, per).contiguous()
    else:
        rows = b + 2 if batch_idx else b
        kc, vc = randn_half(gen, rows, cap, hk, d), randn_half(gen, rows, cap, hk, d)
        if batch_idx:
            idx = torch.randperm(rows, generator=gen)[:b].to(torch.int32)
    if poison_tail and not paged:
        # cache memory past the used length is uninitialised in real use: make it NaN
        for i, n in enumerate(lens):
            row = i if idx is None else int(idx[i])
            kc[row, n + s_new:] = float("nan")
            vc[row, n + s_new:] = float("nan")
    kc_ref, vc_ref = kc.clone(), vc.clone()
    o_ref, lse_ref = orc.kvcache_forward(q, kc_ref, vc_ref, kn, vn, lens_t, idx, table,
                                         d ** -0.5 if scale is None else scale, causal)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    out, lse = flash_attn_with_kvcache(
        q.to(DEV), kcd, vcd, kn.to(DEV) if s_new else None, vn.to(DEV) if s_new else None,
        cache_seqlens=lens_t.to(DEV), cache_batch_idx=None if idx is None else idx.to(DEV),
        block_table=None if table is None else table.to(DEV), softmax_scale=scale, causal=causal,
        num_splits=splits, return_softmax_lse=True)
    assert not torch.isnan(out).any()
    assert err_stats(out, o_ref)[0] <= O_TOL
    assert err_stats(lse, lse_ref)[0] <= LSE_TOL
    # the appended cache is an observable output: bit-exact copies, nothing else touched
    assert torch.equal(torch.nan_to_num(kcd.cpu()), torch.nan_to_num(kc_ref))
    assert torch.equal(torch.nan_to_num(vcd.cpu()), torch.nan_to_num(vc_ref))
    return out, lse


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("h,hk", [(6, 1), (4, 2), (4, 4)])
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 8])
def test_contiguous_decode(ext, d, h, hk, splits):
    _run(3, 1, h, hk, d, 1024, [1, 511, 1000], 0, splits=splits)
    _run(3, 1, h, hk, d, 1024, [0, 511, 1000], 1, splits=splits)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("page", [256, 512, 768, 1024])
@pytest.mark.parametrize("splits", [0, 1, 4, 16])
def test_paged_decode_append(ext, d, page, splits):
    _run(3, 1, 8, 2, d, 4096, [5, 3000, 4095], 1, paged=True, page=page, splits=splits)


@pytest.mark.parametrize("sq,s_new", [(2, 2), (3, 1), (4, 4), (7, 7), (16, 16), (16, 0), (200, 200), (130, 5)])
@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("causal", [False, True])
def test_query_chunks(ext, sq, s_new, paged, causal):
    # (sq * group) <= 16 rows -> split-KV decode kernel; above -> tiled tcgen05 kernel over the cache
    _run(2, sq, 4, 2, 128, 2048, [300, 1500], s_new, paged=paged, splits=0, causal=causal)
    _run(2, sq, 6, 3, 64, 2048, [0, 1800], s_new, paged=paged, splits=2, causal=causal)


def test_cache_batch_idx_and_scale(ext):
    _run(3, 1, 6, 1, 64, 1024, [1, 511, 1000], 1, splits=2, batch_idx=True, scale=0.3)
    _run(2, 7, 6, 3, 64, 1024, [10, 1000], 7, splits=1, batch_idx=True)
    _run(2, 40, 4, 2, 128, 1024, [10, 900], 40, splits=0, batch_idx=True)


def test_uninitialised_cache_tail_is_never_used(ext):
    _run(2, 1, 4, 2, 128, 1024, [100, 777], 1, splits=1, poison_tail=True)
    _run(2, 1, 4, 2, 64, 1024, [100, 777], 1, splits=4, poison_tail=True)
    # query chunks that go through the tiled tcgen05 kernel (more than 16 rows per KV head)
    _run(2, 40, 4, 2, 128, 1024, [100, 777], 40, splits=0, poison_tail=True)
    _run(2, 130, 4, 4, 64, 1024, [3, 500], 130, splits=0, poison_tail=True, causal=False)


def test_int_and_default_cache_seqlens(ext):
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    gen = torch.Generator().manual_seed(1)
    q, kc, vc = randn_half(gen, 2, 1, 4, 64), randn_half(gen, 2, 320, 2, 64), randn_half(gen, 2, 320, 2, 64)
    o_ref, _ = orc.kvcache_forward(q, kc.clone(), vc.clone(), None, None, [200, 200], None, None, None, True)
    out = flash_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), cache_seqlens=200, causal=True)
    assert isinstance(out, torch.Tensor) and err_stats(out, o_ref)[0] <= O_TOL
    o_ref, _ = orc.kvcache_forward(q, kc.clone(), vc.clone(), None, None, [320, 320], None, None, None, True)
    out = flash_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), causal=True)  # whole cache
    assert err_stats(out, o_ref)[0] <= O_TOL


def test_split_counts_agree(ext):
    # the merged result does not depend on the split count beyond fp32 rounding
    outs = [_run(2, 1, 8, 2, 128, 8192, [8000, 4099], 1, paged=True, splits=s)[0] for s in (1, 2, 4, 16, 0)]
    for o in outs[1:]:
        assert err_stats(o, outs[0])[0] <= 1e-3


def test_long_paged_decode(ext):
    # 16k-token paged decode (the reference's largest functional case, test_flash_attn.py:1491-1569)
    _run(2, 1, 8, 2, 128, 16384, [16000, 12345], 1, paged=True, splits=0)


@pytest.mark.parametrize("name", ["fwd_d64_split3", "fwd_d128_decode_split4"])
def test_golden_split_fixtures(ext, name):
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    g = load_golden(name)
    q, k, v = t(g["q"]), t(g["k"]), t(g["v"])
    out, lse = flash_attn_with_kvcache(q.to(DEV), k.to(DEV), v.to(DEV), cache_seqlens=t(g["lens"]).to(DEV),
                                       softmax_scale=float(g["scale"]), causal=bool(g["causal"]),
                                       num_splits=int(g["splits"]), return_softmax_lse=True)
    assert err_stats(out, t(g["out"]))[0] <= O_TOL
    assert err_stats(lse, t(g["lse"]))[0] <= LSE_TOL


@pytest.mark.parametrize("name,paged", [("cache_contiguous", False), ("cache_paged", True)])
def test_golden_cache_append(ext, name, paged):
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    g = load_golden(name)
    kc, vc = t(g["k_cache_before"]).to(DEV), t(g["v_cache_before"]).to(DEV)
    b, hk, d = g["k_new"].shape[0], g["k_new"].shape[2], g["k_new"].shape[3]
    q = torch.zeros(b, 1, hk, d, dtype=torch.half, device=DEV)
    flash_attn_with_kvcache(q, kc, vc, t(g["k_new"]).to(DEV), t(g["v_new"]).to(DEV), cache_seqlens=t(g["lens"]).to(DEV),
                            cache_batch_idx=None if paged else t(g["cache_batch_idx"]).to(DEV),
                            block_table=t(g["block_table"]).to(DEV) if paged else None)
    assert torch.equal(kc.cpu(), t(g["k_cache_after"])) and torch.equal(vc.cpu(), t(g["v_cache_after"]))


def test_cache_batch_idx_out_of_range_is_rejected_on_the_host(ext):
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    q = torch.zeros(1, 1, 2, 64, dtype=torch.half, device=DEV)
    kc = torch.zeros(2, 256, 2, 64, dtype=torch.half, device=DEV)
    with pytest.raises(RuntimeError, match="within cache batch bounds"):
        flash_attn_with_kvcache(q, kc, kc.clone(), cache_seqlens=torch.tensor([4], dtype=torch.int32, device=DEV),
                                cache_batch_idx=torch.tensor([2], dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("splits", [1, 4, 16])
def test_c4_paged_decode_full_size(ext, splits):
    # C4 of the benchmark configs: batch 64, one query token, Hq32 Hkv8 D128, cache_seqlens U[1024, 32768],
    # page 256, 16384-page pool, shuffled block table, in-place append.  Four sequences are checked against
    # the oracle (gathering their pages on the CPU); the appended rows of the pool must hold k/v exactly.
    from flash_attention_turing_b200 import flash_attn_with_kvcache

    b, h, hk, d, page, pages, max_pages = 64, 32, 8, 128, 256, 16384, 129
    gen_c = torch.Generator().manual_seed(1004)
    lens = torch.randint(1024, 32768, (b,), generator=gen_c, dtype=torch.int32)
    perm = torch.randperm(pages, generator=gen_c).to(torch.int32)
    table = torch.zeros(b, max_pages, dtype=torch.int32)
    off = 0
    for i in range(b):
        n = (int(lens[i]) + 1 + page - 1) // page
        table[i, :n] = perm[off:off + n]
        off += n
    gen = torch.Generator(device=DEV).manual_seed(1004)
    kc = torch.randn(pages, page, hk, d, device=DEV, dtype=torch.half, generator=gen)
    vc = torch.randn(pages, page, hk, d, device=DEV, dtype=torch.half, generator=gen)
    q = torch.randn(b, 1, h, d, device=DEV, dtype=torch.half, generator=gen)
    kn = torch.randn(b, 1, hk, d, device=DEV, dtype=torch.half, generator=gen)
    vn = torch.randn(b, 1, hk, d, device=DEV, dtype=torch.half, generator=gen)
    out, lse = flash_attn_with_kvcache(q, kc, vc, kn, vn, cache_seqlens=lens.to(DEV), block_table=table.to(DEV),
                                       causal=True, num_splits=splits, return_softmax_lse=True)
    for i in (0, 17, 40, 63):
        n_tok = int(lens[i]) + 1
        ids = table[i, : (n_tok + page - 1) // page].to(DEV).long()
        ks = kc[ids].reshape(-1, hk, d)[:n_tok].cpu()
        vs = vc[ids].reshape(-1, hk, d)[:n_tok].cpu()
        assert torch.equal(ks[-1], kn[i, 0].cpu()) and torch.equal(vs[-1], vn[i, 0].cpu())  # appended in place
        o_ref, lse_ref = orc.attention_forward_one(q[i].cpu(), ks, vs, d ** -0.5, True)
        assert err_stats(out[i], o_ref)[0] <= O_TOL
        assert err_stats(lse[i], lse_ref)[0] <= LSE_TOL


def test_device_side_capacity_clamp_without_host_check(ext):
    # With the host-side capacity check switched off (no device synchronisation per call) an oversized
    # length must neither read nor write out of bounds: it is clamped to the capacity on the device, the
    # result equals the one for the clamped length, and bit 1 of the status word reports the clamp.
    from flash_attention_turing_b200 import flash_attention_interface as iface

    gen = torch.Generator().manual_seed(4)
    b, h, hk, d, page, per = 2, 4, 2, 128, 256, 2
    kc, vc = randn_half(gen, b * per, page, hk, d), randn_half(gen, b * per, page, hk, d)
    table = torch.arange(b * per, dtype=torch.int32).view(b, per)
    q = randn_half(gen, b, 1, h, d)
    lens_bad = torch.tensor([300, 9999], dtype=torch.int32)       # capacity is 512 tokens per sequence
    lens_ok = torch.tensor([300, 512], dtype=torch.int32)
    o_ref, _ = orc.kvcache_forward(q, kc.clone(), vc.clone(), None, None, lens_ok, None, table, None, True)
    iface.HOST_CAPACITY_CHECK = False
    try:
        out = iface.flash_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), cache_seqlens=lens_bad.to(DEV),
                                            block_table=table.to(DEV), causal=True, num_splits=2)
        status = ext.device_status(True)
    finally:
        iface.HOST_CAPACITY_CHECK = True
    assert status == 2
    assert err_stats(out, o_ref)[0] <= O_TOL
    with pytest.raises(ValueError, match="cache capacity is insufficient"):
        iface.flash_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), cache_seqlens=lens_bad.to(DEV),
                                      block_table=table.to(DEV), causal=True)
