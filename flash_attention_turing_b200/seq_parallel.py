"""Sequence-sharded forward and backward: each rank holds one contiguous shard of K/V, attends ALL
queries against it, and the partial (O, LSE) of the ranks are merged with the split-KV log-sum-exp
combine.  In the backward every rank obtains dK/dV of its shard completely and its keys' share of dQ;
the shares are summed across the ranks.

This is the one place of the attention path that has a real exchange step.  The reference has no
multi-GPU code; the merge is its split-KV combine (``kvcache_combine_kernel``,
``csrc/flash_attn/src/kvcache_native.cu:676-729`` of Cy-47/flash-attention-turing) with one split per
rank.  Plumbing is ``torch.distributed`` (NCCL over NVLink on GPUs; gloo in the CPU tests):

    rank r:  partial_r = attention(q[all rows], k[shard r], v[shard r])        (local kernels)
    all_to_all_single: query-row slice j of every rank's partial -> rank j       (one collective)
    rank j:  out[slice j] = combine(partials of slice j)                         (fa_combine)

    backward, rank r:  dq_share_r, dk[shard r], dv[shard r] = backward(q, k[shard r], v[shard r],
                                                   merged out, merged lse, dout)   (local kernels)
    all_to_all_single: query-row slice j of every rank's dq share -> rank j        (one collective)
    rank j:  dq[slice j] = sum of the shares of slice j                            (fa_sum_gather)

With ``layout="zigzag"`` rank r holds chunks r and 2*world-1-r of 2*world equal chunks, which gives every
rank the same amount of causal work (a contiguous range gives the last rank 2*world-1 times the work of
the first); the rank merges (adds) the results of its two chunks locally before the exchange.

In these paths no kernel reads peer memory: the collective lands the partials in local memory first.
The ``*_p2p`` variants replace the collective by ONE kernel that reads the peers' buffers in place.

``partial_attention`` and ``merge_partials`` take the kernels as injectable callables so that the
exchange logic can be exercised by CPU ranks in the tests (with the oracle as the kernel stand-in);
by default they call the CUDA library and fail if it is missing.

On CUDA tensors with the default kernels the public functions take a path without eager tensor arithmetic:
ONE forward (backward) launch per K/V chunk with an explicit causal diagonal (``causal_shift``), writing
straight into row blocks of the exchange buffers; query rows a chunk cannot see are marked by LSE = -inf
(forward) or by a per-part first valid row (backward) and are never read by the merge kernels; for one
sequence (batch 1) the all-to-all sends the partial as it lies in memory.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

FwdFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, float, bool], Tuple[torch.Tensor, torch.Tensor]]
# (q, k, v, out, lse, dout, scale, causal) -> (dq, dk, dv), from SAVED out / lse as the extension's bwd does
BwdFn = Callable[..., Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]
SumFn = Callable[[torch.Tensor], torch.Tensor]  # (world, b, sl, h, d) shares -> (b, sl, h, d) sum
CombineFn = Callable[[torch.Tensor, torch.Tensor, int, int, int], Tuple[torch.Tensor, torch.Tensor]]


def _default_fwd(q, k, v, scale, causal):
    from . import _ext

    return _ext.load().fwd(q, k, v, scale, causal)


def _default_combine(o_accum, lse_accum, b, sq, h):
    from . import _ext

    return _ext.load().combine(o_accum, lse_accum, b, sq, h)


def _default_bwd(q, k, v, out, lse, dout, scale, causal):
    from . import _ext

    return _ext.load().bwd(q, k, v, out, lse, dout, scale, causal)


def _default_sum(shares):
    from . import _ext

    return _ext.load().sum_gather(list(shares.unbind(0)), 0, shares.shape[2])


def _default_merge2(o_parts, lse_parts):
    from . import _ext

    return _ext.load().combine_gather(list(o_parts), list(lse_parts), 0, o_parts[0].shape[1])


def _default_add2(parts):
    from . import _ext

    return _ext.load().sum_gather(list(parts), 0, parts[0].shape[1])


def _check_layout(layout: str) -> bool:
    if layout not in ("contiguous", "zigzag"):
        raise ValueError("layout must be 'contiguous' or 'zigzag'")
    return layout == "zigzag"


def shard_chunks(rank: int, world: int, seqlen: int, layout: str = "contiguous"):
    """Key ranges [(begin, end), ...] of rank ``rank``: one contiguous range, or the two zig-zag chunks."""
    if _check_layout(layout):
        if seqlen % (2 * world) != 0:
            raise ValueError("seqlen_k must be divisible by twice the number of ranks for the zigzag layout")
        c = seqlen // (2 * world)
        return [(rank * c, (rank + 1) * c), ((2 * world - 1 - rank) * c, (2 * world - rank) * c)]
    if seqlen % world != 0:
        raise ValueError("seqlen_k must be divisible by the number of ranks")
    c = seqlen // world
    return [(rank * c, (rank + 1) * c)]


def shard_kv(x: torch.Tensor, rank: int, world: int, layout: str = "contiguous") -> torch.Tensor:
    """The rows of x (b, s, h_k, d) that rank ``rank`` holds, concatenated in the order of ``shard_chunks``."""
    return torch.cat([x[:, b:e] for b, e in shard_chunks(rank, world, x.shape[1], layout)], dim=1).contiguous()


def partial_attention(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, key_offset: int,
                      softmax_scale: float, causal: bool, fwd: Optional[FwdFn] = None,
                      out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of all queries against one K/V shard that starts at global key index ``key_offset``.

    q (b, s, h, d); k_shard / v_shard (b, s_shard, h_k, d).  Returns the shard-normalised partial output
    (b, s, h, d) in q's dtype and the partial LSE (b, h, s) fp32, ``-inf`` for query rows that see no key of
    the shard.  Causal (global key j visible to query i iff j <= i, seqlen_q == seqlen_k): rows before
    the shard see nothing, the ``s_shard`` rows on the shard's diagonal are a square causal problem, the
    rows after it see the whole shard -- two launches of the ordinary forward kernel.
    """
    fwd = fwd or _default_fwd
    b, s, h, d = q.shape
    s_shard = k_shard.shape[1]
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((b, h, s), dtype=torch.float32, device=q.device)
    if s_shard == 0 or causal:
        out.zero_()
        lse.fill_(float("-inf"))
    if s_shard == 0:
        return out, lse
    if not causal:
        o, l = fwd(q, k_shard, v_shard, softmax_scale, False)
        out.copy_(o)
        lse.copy_(l)
        return out, lse
    lo = min(key_offset, s)
    mid = min(key_offset + s_shard, s)
    if mid > lo:  # diagonal block: square causal problem
        o, l = fwd(q[:, lo:mid], k_shard[:, : mid - lo], v_shard[:, : mid - lo], softmax_scale, True)
        out[:, lo:mid] = o
        lse[:, :, lo:mid] = l
    if s > mid:  # rows below the diagonal block see the whole shard
        o, l = fwd(q[:, mid:], k_shard, v_shard, softmax_scale, False)
        out[:, mid:] = o
        lse[:, :, mid:] = l
    return out, lse


def _fast(q: torch.Tensor, *injected) -> bool:
    """The copy-free CUDA path applies when no stand-in kernel was injected."""
    return q.is_cuda and all(x is None for x in injected)


def chunk_first_rows(world: int, seqlen: int, layout: str, causal: bool):
    """For every (rank, chunk) in the order the parts are merged: the first query row that sees a key of the
    chunk (0 without a causal mask)."""
    rows = []
    for r in range(world):
        for kb, _ in shard_chunks(r, world, seqlen, layout):
            rows.append(min(kb, seqlen) if causal else 0)
    return rows


def rank_partials_inplace(q, k_shard, v_shard, rank: int, world: int, softmax_scale: float, causal: bool,
                          layout: str, out_bufs: torch.Tensor, lse_bufs: torch.Tensor) -> None:
    """One forward launch per chunk of this rank, written in place: out_bufs (chunks, b, s, h, d) and lse_bufs
    (chunks, b, h, s).  Chunk c attends query rows [first, s) -- the rows that can see it -- against its keys
    with the diagonal at key 0 <-> row `first` (causal_shift = 0); rows below `first` get LSE = -inf and their
    O rows are left untouched (the merge kernels do not read them)."""
    from . import _ext

    ext = _ext.load()
    s = q.shape[1]
    local = 0
    for ci, (kb, ke) in enumerate(shard_chunks(rank, world, s, layout)):
        c = ke - kb
        ks, vs = k_shard[:, local:local + c], v_shard[:, local:local + c]
        local += c
        first = min(kb, s) if causal else 0
        if first > 0:
            lse_bufs[ci][:, :, :first].fill_(float("-inf"))
        if first < s:
            ext.fwd(q[:, first:], ks, vs, softmax_scale, causal, out=out_bufs[ci][:, first:],
                    lse=lse_bufs[ci][:, :, first:], causal_shift=0 if causal else None)


def rank_backward_inplace(q, k_shard, v_shard, out, lse, dout, rank: int, world: int, softmax_scale: float,
                          causal: bool, layout: str, dq_bufs: torch.Tensor, dk_shard: torch.Tensor,
                          dv_shard: torch.Tensor) -> None:
    """One backward launch per chunk of this rank: the chunk's dQ share goes to rows [first, s) of dq_bufs[c]
    (chunks, b, s, h, d) -- rows below `first` are left untouched, the reduction skips them -- and its dK, dV
    to the chunk's rows of dk_shard / dv_shard."""
    from . import _ext

    ext = _ext.load()
    s = q.shape[1]
    local = 0
    for ci, (kb, ke) in enumerate(shard_chunks(rank, world, s, layout)):
        c = ke - kb
        first = min(kb, s) if causal else 0
        sl = slice(local, local + c)
        local += c
        if first >= s:
            dk_shard[:, sl].zero_()
            dv_shard[:, sl].zero_()
            continue
        ext.bwd(q[:, first:], k_shard[:, sl], v_shard[:, sl], out[:, first:], lse[:, :, first:], dout[:, first:],
                softmax_scale, causal, dq=dq_bufs[ci][:, first:], dk=dk_shard[:, sl], dv=dv_shard[:, sl],
                causal_shift=0 if causal else None)


def _exchange_rows(x: torch.Tensor, world: int, group) -> torch.Tensor:
    """all_to_all of the query-row slices of x (b, s, h, d): returns (world, b, s / world, h, d), entry r = this
    rank's slice as rank r holds it.  For one sequence the slices are sent as they lie in memory."""
    b, s, h, d = x.shape
    sl = s // world
    send = x.view(world, 1, sl, h, d) if b == 1 else x.view(b, world, sl, h, d).transpose(0, 1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def merge_partials(o_part: torch.Tensor, lse_part: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                   combine: Optional[CombineFn] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exchange and merge.  o_part (b, s, h, d), lse_part (b, h, s) are this rank's partials for ALL query
    rows; s must be divisible by the world size.  Returns this rank's slice of the final result:
    out (b, s / world, h, d) in o_part's dtype and lse (b, h, s / world) fp32."""
    world = dist.get_world_size(group)
    b, s, h, d = o_part.shape
    if s % world != 0:
        raise ValueError("seqlen_q must be divisible by the number of ranks")
    sl = s // world
    if _fast(o_part, combine):
        # the received slices are fp16 partials in the forward's own layout: fa_combine_gather merges them as
        # they are (no conversion, no transposition of O); only the small LSE tensor is re-laid
        from . import _ext

        o_recv = _exchange_rows(o_part, world, group)
        l_send = lse_part.view(b, h, world, sl).permute(2, 0, 1, 3).contiguous()
        l_recv = torch.empty_like(l_send)
        dist.all_to_all_single(l_recv, l_send, group=group)
        out, lse = _ext.load().combine_gather(list(o_recv.unbind(0)), list(l_recv.unbind(0)), 0, sl)
        return out, lse
    combine = combine or _default_combine
    # send buffers: slice j of the query rows, laid out (b, h, sl, d) so that the received block of every
    # source rank is already in the (rows = (b, h, sl), d) order the combine kernel reads
    o_send = o_part.view(b, world, sl, h, d).permute(1, 0, 3, 2, 4).contiguous()      # (world, b, h, sl, d)
    l_send = lse_part.view(b, h, world, sl).permute(2, 0, 1, 3).contiguous()          # (world, b, h, sl)
    o_recv = torch.empty_like(o_send)
    l_recv = torch.empty_like(l_send)
    dist.all_to_all_single(o_recv, o_send, group=group)
    dist.all_to_all_single(l_recv, l_send, group=group)
    rows = b * h * sl
    out, lse = combine(o_recv.view(world, rows, d).float(), l_recv.view(world, rows), b, sl, h)
    return out.to(o_part.dtype), lse


def rank_partial(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, rank: int, world: int,
                 softmax_scale: float, causal: bool, layout: str = "contiguous", fwd: Optional[FwdFn] = None,
                 merge2=None, out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None):
    """This rank's partial (O, LSE) for all query rows: ``partial_attention`` on its range, or on each of its
    two zig-zag chunks followed by a local log-sum-exp merge of the two (``fa_combine_gather`` with two
    local parts by default)."""
    if not _check_layout(layout):
        return partial_attention(q, k_shard, v_shard, rank * k_shard.shape[1], softmax_scale, causal, fwd, out, lse)
    c = k_shard.shape[1] // 2
    parts = [partial_attention(q, k_shard[:, i * c:(i + 1) * c], v_shard[:, i * c:(i + 1) * c], off, softmax_scale,
                               causal, fwd)
             for i, off in enumerate((rank * c, (2 * world - 1 - rank) * c))]
    o, l = (merge2 or _default_merge2)([p[0] for p in parts], [p[1] for p in parts])
    # rows that saw no key in either chunk: the merge reports LSE 0 there, the exchange wants -inf
    dead = torch.isinf(parts[0][1]) & torch.isinf(parts[1][1])
    l = torch.where(dead, torch.full_like(l, float("-inf")), l)
    if out is not None:
        out.copy_(o)
        lse.copy_(l)
        return out, lse
    return o.to(q.dtype), l


def sequence_parallel_forward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                              softmax_scale: Optional[float] = None, causal: bool = False,
                              group: Optional[dist.ProcessGroup] = None, gather_output: bool = False,
                              fwd: Optional[FwdFn] = None, combine: Optional[CombineFn] = None,
                              layout: str = "contiguous", merge2=None):
    """Forward with K/V sharded over the ranks of ``group`` (``shard_kv``: equal contiguous ranges, rank r
    holding keys [r * s_shard, (r + 1) * s_shard), or zig-zag chunk pairs); q is replicated.  Returns
    (out, lse) for this rank's query-row slice, or for all rows when ``gather_output`` is set."""
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
    if _fast(q, fwd, combine, merge2):
        b, s, h, d = q.shape
        nch = 2 if _check_layout(layout) else 1
        o_bufs = torch.empty((nch, b, s, h, d), dtype=q.dtype, device=q.device)
        l_bufs = torch.empty((nch, b, h, s), dtype=torch.float32, device=q.device)
        rank_partials_inplace(q, k_shard, v_shard, rank, world, scale, causal, layout, o_bufs, l_bufs)
        if nch == 2:  # the two zig-zag chunks are merged locally, so that one partial travels
            o_part, lse_part = _default_merge2(list(o_bufs.unbind(0)), list(l_bufs.unbind(0)))
            dead = torch.isinf(l_bufs[0]) & torch.isinf(l_bufs[1])
            lse_part = torch.where(dead, torch.full_like(lse_part, float("-inf")), lse_part)
        else:
            o_part, lse_part = o_bufs[0], l_bufs[0]
    else:
        o_part, lse_part = rank_partial(q, k_shard, v_shard, rank, world, scale, causal, layout, fwd, merge2)
    out, lse = merge_partials(o_part, lse_part, group, combine)
    if not gather_output:
        return out, lse
    outs = [torch.empty_like(out) for _ in range(world)]
    lses = [torch.empty_like(lse) for _ in range(world)]
    dist.all_gather(outs, out, group=group)
    dist.all_gather(lses, lse, group=group)
    return torch.cat(outs, dim=1), torch.cat(lses, dim=2)


# ------------------------------------------------------------------------------------------------
# Fused exchange + merge: every rank reads the other ranks' partials directly from their memory
# ------------------------------------------------------------------------------------------------
_P2P_BUFFERS: "OrderedDict" = None  # type: ignore[assignment]
_P2P_MAX_SHAPES = 4  # symmetric buffers are kept for the most recently used shapes only


def _p2p_buffers(shape_o, shape_l, dtype, device, group):
    """Symmetric-memory buffers for the partial (O, LSE) of one problem shape, allocated and exchanged once
    per (shape, group) and reused; the least recently used shape is dropped beyond _P2P_MAX_SHAPES.
    Returns (o_buf, lse_buf, handle_o, handle_l).  Collective: every rank of the group must call it with the
    same arguments."""
    import torch.distributed._symmetric_memory as symm_mem
    from collections import OrderedDict

    global _P2P_BUFFERS
    if _P2P_BUFFERS is None:
        _P2P_BUFFERS = OrderedDict()
    group = group or dist.group.WORLD
    key = (tuple(shape_o), tuple(shape_l), dtype, str(device), group.group_name)
    if key in _P2P_BUFFERS:
        _P2P_BUFFERS.move_to_end(key)
        return _P2P_BUFFERS[key]
    o_buf = symm_mem.empty(*shape_o, dtype=dtype, device=device)
    l_buf = symm_mem.empty(*shape_l, dtype=torch.float32, device=device)
    _P2P_BUFFERS[key] = (o_buf, l_buf, symm_mem.rendezvous(o_buf, group.group_name),
                         symm_mem.rendezvous(l_buf, group.group_name))
    while len(_P2P_BUFFERS) > _P2P_MAX_SHAPES:
        _P2P_BUFFERS.popitem(last=False)
    return _P2P_BUFFERS[key]


def peer_memory_available(shape_o, shape_l, dtype, device, group: Optional[dist.ProcessGroup] = None) -> bool:
    """Collective.  True iff EVERY rank of the group could allocate and map the symmetric buffers for this
    problem shape.  The ranks agree on the answer with a host-side all-reduce, so that either all of them
    take a ``*_p2p`` path (which waits for its peers on the device) or none does."""
    ok = 1
    try:
        _p2p_buffers(shape_o, shape_l, dtype, device, group)
    except (ImportError, RuntimeError, AttributeError) as exc:
        ok = 0
        _last_p2p_error[0] = f"{type(exc).__name__}: {exc}"
    flag = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


def peer_memory_available_for(q: torch.Tensor, layout: str = "contiguous",
                              group: Optional[dist.ProcessGroup] = None) -> bool:
    """Collective.  ``peer_memory_available`` for the buffers the ``*_p2p`` functions use with this q and layout."""
    b, s, h, d = q.shape
    nch = 2 if _check_layout(layout) else 1
    return peer_memory_available((nch, b, s, h, d), (nch, b, h, s), q.dtype, q.device, group)


_last_p2p_error = [""]


def last_peer_memory_error() -> str:
    """Why peer_memory_available() last said no on this rank ("" if it did not)."""
    return _last_p2p_error[0]


def owned_rows(rank: int, world: int, seqlen: int, row_layout: str = "contiguous"):
    """The query rows whose final result a rank produces, as (begin, end) ranges in output order: one contiguous
    slice, or with row_layout="zigzag" the rows of chunks ``rank`` and ``2 * world - 1 - rank`` of 2 * world equal
    chunks.  Under a causal mask the late rows see every K/V chunk and the early rows one or two, so with
    contiguous slices the last rank merges (and fetches over NVLink) almost twice the average and the first
    almost nothing; the zig-zag rows give every rank the same amount."""
    if _check_layout(row_layout):
        return shard_chunks(rank, world, seqlen, "zigzag")
    sl = seqlen // world
    return [(rank * sl, (rank + 1) * sl)]


def gather_owned_rows(x: torch.Tensor, rank: int, world: int, row_layout: str = "contiguous", dim: int = 1):
    """The rows of a full-length tensor that ``owned_rows`` assigns to a rank, in output order."""
    return torch.cat([x.narrow(dim, b, e - b) for b, e in owned_rows(rank, world, x.shape[dim], row_layout)], dim=dim)


def sequence_parallel_forward_p2p(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                                  softmax_scale: Optional[float] = None, causal: bool = False,
                                  group: Optional[dist.ProcessGroup] = None, layout: str = "contiguous",
                                  row_layout: str = "contiguous"):
    """Same result as ``sequence_parallel_forward`` (this rank's query-row slice), but without the
    all-to-all: the partials are written into symmetric memory, a device-side barrier orders the ranks,
    and ONE kernel (``fa_combine_gather``) reads the query-row slice of every rank's partial straight from
    that rank's HBM over NVLink (plain loads, no multicast) and merges it.  Needs
    ``torch.distributed._symmetric_memory``; raises if the peers' memory cannot be mapped."""
    from . import _ext

    ext = _ext.load()
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    b, s, h, d = q.shape
    if s % world != 0:
        raise ValueError("seqlen_q must be divisible by the number of ranks")
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    # Everything that can fail on the host -- allocation, rendezvous, mapping the peers' buffers, the local
    # kernels' argument checks -- happens before the first device-side barrier; between the two barriers the
    # merge runs under try/finally, so a rank that fails there still releases its peers.
    nch = 2 if _check_layout(layout) else 1
    if nch * world > 16:
        raise ValueError("at most 16 K/V chunks in total (8 ranks with the zigzag layout)")
    shape_o, shape_l = (nch, b, s, h, d), (nch, b, h, s)
    o_buf, l_buf, hdl_o, hdl_l = _p2p_buffers(shape_o, shape_l, q.dtype, q.device, group)
    o_parts = [x for r in range(world) for x in hdl_o.get_buffer(r, shape_o, q.dtype).unbind(0)]
    l_parts = [x for r in range(world) for x in hdl_l.get_buffer(r, shape_l, torch.float32).unbind(0)]
    # one launch per chunk, written straight into the symmetric buffers; each chunk of each rank is one part of
    # the merge (no local pre-merge of the two zig-zag chunks), dead rows are skipped through LSE = -inf
    rank_partials_inplace(q, k_shard, v_shard, rank, world, scale, causal, layout, o_buf, l_buf)
    mine = owned_rows(rank, world, s, row_layout)  # (see there; output rows in this order)
    hdl_o.barrier(channel=0)  # every rank's partial is complete and visible
    try:
        res = [ext.combine_gather(o_parts, l_parts, rb, re - rb) for rb, re in mine]
    finally:
        hdl_o.barrier(channel=1)  # nobody overwrites a partial that a peer is still reading
    if len(res) == 1:
        return res[0]
    return torch.cat([r[0] for r in res], dim=1), torch.cat([r[1] for r in res], dim=2)


# ------------------------------------------------------------------------------------------------
# Backward
# ------------------------------------------------------------------------------------------------
def partial_backward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, out: torch.Tensor,
                     lse: torch.Tensor, dout: torch.Tensor, key_offset: int, softmax_scale: float, causal: bool,
                     bwd: Optional[BwdFn] = None, dq_share: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of all queries against one K/V shard that starts at global key index ``key_offset``.

    ``out`` (b, s, h, d) and ``lse`` (b, h, s) are the MERGED results of the forward for all query rows,
    ``dout`` the gradient of ``out``.  Because the kernels recompute P = exp(scale S - lse) from the saved
    lse and D = rowsum(dO o out) from the saved out, running them on the shard's keys alone gives the exact
    dK, dV of the shard and the shard's share of dQ.  Returns (dq_share (b, s, h, d), dk_shard, dv_shard) in
    the input dtype; dq_share is zero for rows that see no key of the shard.  Causal: the same two launches
    as in ``partial_attention`` (square causal problem on the shard's diagonal, dense rectangle below it),
    with dK / dV of the two added in fp32."""
    bwd = bwd or _default_bwd
    b, s, h, d = q.shape
    s_shard = k_shard.shape[1]
    if dq_share is None:
        dq_share = torch.empty_like(q)
    if s_shard == 0:
        dq_share.zero_()
        return dq_share, torch.zeros_like(k_shard), torch.zeros_like(v_shard)
    if not causal:
        dq, dk, dv = bwd(q, k_shard, v_shard, out, lse.contiguous(), dout, softmax_scale, False)
        dq_share.copy_(dq)
        return dq_share, dk, dv
    lo = min(key_offset, s)
    mid = min(key_offset + s_shard, s)
    dq_share[:, :lo].zero_()
    dk = torch.zeros(k_shard.shape, dtype=torch.float32, device=k_shard.device)
    dv = torch.zeros(v_shard.shape, dtype=torch.float32, device=v_shard.device)
    if mid > lo:  # diagonal block: square causal problem
        n = mid - lo
        dq, dk_a, dv_a = bwd(q[:, lo:mid], k_shard[:, :n], v_shard[:, :n], out[:, lo:mid],
                             lse[:, :, lo:mid].contiguous(), dout[:, lo:mid], softmax_scale, True)
        dq_share[:, lo:mid] = dq
        dk[:, :n] += dk_a.float()
        dv[:, :n] += dv_a.float()
    if s > mid:  # rows below the diagonal block see the whole shard
        dq, dk_b, dv_b = bwd(q[:, mid:], k_shard, v_shard, out[:, mid:], lse[:, :, mid:].contiguous(),
                             dout[:, mid:], softmax_scale, False)
        dq_share[:, mid:] = dq
        dk += dk_b.float()
        dv += dv_b.float()
    return dq_share, dk.to(k_shard.dtype), dv.to(v_shard.dtype)


def rank_backward(q, k_shard, v_shard, out, lse, dout, rank: int, world: int, softmax_scale: float, causal: bool,
                  layout: str = "contiguous", bwd: Optional[BwdFn] = None, add2=None,
                  dq_share: Optional[torch.Tensor] = None):
    """This rank's (dq share for all rows, dk_shard, dv_shard): ``partial_backward`` on its range, or on each
    of its two zig-zag chunks with the two dQ shares added (``fa_sum_gather`` with two local parts by
    default) and dK / dV concatenated in shard order."""
    if not _check_layout(layout):
        return partial_backward(q, k_shard, v_shard, out, lse, dout, rank * k_shard.shape[1], softmax_scale, causal,
                                bwd, dq_share)
    c = k_shard.shape[1] // 2
    res = [partial_backward(q, k_shard[:, i * c:(i + 1) * c], v_shard[:, i * c:(i + 1) * c], out, lse, dout, off,
                            softmax_scale, causal, bwd)
           for i, off in enumerate((rank * c, (2 * world - 1 - rank) * c))]
    dq = (add2 or _default_add2)([r[0] for r in res])
    if dq_share is not None:
        dq_share.copy_(dq)
        dq = dq_share
    return dq.to(q.dtype), torch.cat([r[1] for r in res], dim=1), torch.cat([r[2] for r in res], dim=1)


def reduce_dq_shares(dq_share: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                     sum_parts: Optional[SumFn] = None) -> torch.Tensor:
    """Exchange and sum.  dq_share (b, s, h, d) is this rank's share for ALL query rows; returns this rank's
    query-row slice of the sum, (b, s / world, h, d).  The shares travel in their own dtype (half the bytes
    of an fp32 reduce-scatter) and are added in fp32 on arrival."""
    sum_parts = sum_parts or _default_sum
    world = dist.get_world_size(group)
    b, s, h, d = dq_share.shape
    if s % world != 0:
        raise ValueError("seqlen_q must be divisible by the number of ranks")
    sl = s // world
    send = dq_share.view(b, world, sl, h, d).transpose(0, 1).contiguous()  # (world, b, sl, h, d)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return sum_parts(recv)


def sequence_parallel_backward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, out: torch.Tensor,
                               lse: torch.Tensor, dout: torch.Tensor, softmax_scale: Optional[float] = None,
                               causal: bool = False, group: Optional[dist.ProcessGroup] = None,
                               bwd: Optional[BwdFn] = None, sum_parts: Optional[SumFn] = None,
                               layout: str = "contiguous", add2=None):
    """Backward of ``sequence_parallel_forward``.  q, dout and the merged out (b, s, h, d) / lse (b, h, s) are
    replicated (all query rows on every rank, e.g. from ``gather_output=True``); K/V are sharded as in the
    forward.  Returns (dq for this rank's query-row slice (b, s / world, h, d), dk_shard, dv_shard)."""
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
    if _fast(q, bwd, sum_parts, add2):
        from . import _ext

        ext = _ext.load()
        b, s, h, d = q.shape
        if s % world != 0:
            raise ValueError("seqlen_q must be divisible by the number of ranks")
        sl = s // world
        nch = 2 if _check_layout(layout) else 1
        dq_bufs = torch.empty((nch, b, s, h, d), dtype=q.dtype, device=q.device)
        dk, dv = torch.empty_like(k_shard), torch.empty_like(v_shard)
        rank_backward_inplace(q, k_shard, v_shard, out, lse, dout, rank, world, scale, causal, layout, dq_bufs, dk, dv)
        firsts = chunk_first_rows(world, s, layout, causal)
        mine = firsts[rank * nch:(rank + 1) * nch]
        # the two zig-zag shares are added locally (rows neither chunk sees come out as zero), then ONE share travels
        share = ext.sum_gather(list(dq_bufs.unbind(0)), 0, s, mine) if nch == 2 else dq_bufs[0]
        recv = _exchange_rows(share, world, group)  # (world, b, sl, h, d)
        # rank r's share is valid from the first row its lowest chunk sees, here in the coordinates of this slice
        first_in_slice = [max(0, min(sl, min(firsts[r * nch:(r + 1) * nch]) - rank * sl)) for r in range(world)]
        return ext.sum_gather(list(recv.unbind(0)), 0, sl, first_in_slice), dk, dv
    dq_share, dk, dv = rank_backward(q, k_shard, v_shard, out, lse, dout, rank, world, scale, causal, layout, bwd,
                                     add2)
    return reduce_dq_shares(dq_share, group, sum_parts), dk, dv


def sequence_parallel_backward_p2p(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, out: torch.Tensor,
                                   lse: torch.Tensor, dout: torch.Tensor, softmax_scale: Optional[float] = None,
                                   causal: bool = False, group: Optional[dist.ProcessGroup] = None,
                                   layout: str = "contiguous", row_layout: str = "contiguous"):
    """Same result as ``sequence_parallel_backward`` without the all-to-all: the dQ shares are written into
    symmetric memory, a device-side barrier orders the ranks, and ONE kernel (``fa_sum_gather``) reads the
    query-row slice of every rank's share straight from that rank's HBM over NVLink (plain loads, no
    multicast) and adds them."""
    from . import _ext

    ext = _ext.load()
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    b, s, h, d = q.shape
    if s % world != 0:
        raise ValueError("seqlen_q must be divisible by the number of ranks")
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    nch = 2 if _check_layout(layout) else 1
    if nch * world > 16:
        raise ValueError("at most 16 K/V chunks in total (8 ranks with the zigzag layout)")
    shape_o, shape_l = (nch, b, s, h, d), (nch, b, h, s)
    buf, _, hdl, _ = _p2p_buffers(shape_o, shape_l, q.dtype, q.device, group)
    parts = [x for r in range(world) for x in hdl.get_buffer(r, shape_o, q.dtype).unbind(0)]
    dk, dv = torch.empty_like(k_shard), torch.empty_like(v_shard)
    # one launch per chunk; the dQ share of every chunk of every rank is one part of the sum, valid from the
    # first row that sees the chunk (rows below are neither written here nor read over NVLink there)
    rank_backward_inplace(q, k_shard, v_shard, out, lse, dout, rank, world, scale, causal, layout, buf, dk, dv)
    mine = owned_rows(rank, world, s, row_layout)
    firsts = chunk_first_rows(world, s, layout, causal)
    hdl.barrier(channel=0)  # every rank's share is complete and visible
    try:
        res = [ext.sum_gather(parts, rb, re - rb, firsts) for rb, re in mine]
    finally:
        hdl.barrier(channel=1)  # nobody overwrites a share that a peer is still reading
    return (res[0] if len(res) == 1 else torch.cat(res, dim=1)), dk, dv
