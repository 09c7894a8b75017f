"""Sequence-sharded forward: each rank holds one contiguous shard of K/V, attends ALL queries against
it, and the partial (O, LSE) of the ranks are merged with the split-KV log-sum-exp combine.

This is the one place of the attention path that has a real exchange step.  The reference has no
multi-GPU code; the merge is its split-KV combine (``kvcache_combine_kernel``,
``csrc/flash_attn/src/kvcache_native.cu:676-729`` of Cy-47/flash-attention-turing) with one split per
rank.  Plumbing is ``torch.distributed`` (NCCL over NVLink on GPUs; gloo in the CPU tests):

    rank r:  partial_r = attention(q[all rows], k[shard r], v[shard r])        (local kernels)
    all_to_all_single: query-row slice j of every rank's partial -> rank j       (one collective)
    rank j:  out[slice j] = combine(partials of slice j)                         (fa_combine)

No peer memory is read by any kernel: the collective lands the partials in local memory first.

``partial_attention`` and ``merge_partials`` take the kernels as injectable callables so that the
exchange logic can be exercised by CPU ranks in the tests (with the oracle as the kernel stand-in);
by default they call the CUDA library and fail if it is missing.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

FwdFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, float, bool], Tuple[torch.Tensor, torch.Tensor]]
CombineFn = Callable[[torch.Tensor, torch.Tensor, int, int, int], Tuple[torch.Tensor, torch.Tensor]]


def _default_fwd(q, k, v, scale, causal):
    from . import _ext

    return _ext.load().fwd(q, k, v, scale, causal)


def _default_combine(o_accum, lse_accum, b, sq, h):
    from . import _ext

    return _ext.load().combine(o_accum, lse_accum, b, sq, h)


def partial_attention(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, key_offset: int,
                      softmax_scale: float, causal: bool, fwd: Optional[FwdFn] = None
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
    out = torch.zeros_like(q)
    lse = torch.full((b, h, s), float("-inf"), dtype=torch.float32, device=q.device)
    if s_shard == 0:
        return out, lse
    if not causal:
        o, l = fwd(q, k_shard, v_shard, softmax_scale, False)
        return o, l
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


def merge_partials(o_part: torch.Tensor, lse_part: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                   combine: Optional[CombineFn] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exchange and merge.  o_part (b, s, h, d), lse_part (b, h, s) are this rank's partials for ALL query
    rows; s must be divisible by the world size.  Returns this rank's slice of the final result:
    out (b, s / world, h, d) in o_part's dtype and lse (b, h, s / world) fp32."""
    combine = combine or _default_combine
    world = dist.get_world_size(group)
    b, s, h, d = o_part.shape
    if s % world != 0:
        raise ValueError("seqlen_q must be divisible by the number of ranks")
    sl = s // world
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


def sequence_parallel_forward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                              softmax_scale: Optional[float] = None, causal: bool = False,
                              group: Optional[dist.ProcessGroup] = None, gather_output: bool = False,
                              fwd: Optional[FwdFn] = None, combine: Optional[CombineFn] = None):
    """Forward with K/V sharded over the ranks of ``group`` by contiguous sequence ranges of equal length
    (rank r holds keys [r * s_shard, (r + 1) * s_shard)); q is replicated.  Returns (out, lse) for this
    rank's query-row slice, or for all rows when ``gather_output`` is set."""
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
    o_part, lse_part = partial_attention(q, k_shard, v_shard, rank * k_shard.shape[1], scale, causal, fwd)
    out, lse = merge_partials(o_part, lse_part, group, combine)
    if not gather_output:
        return out, lse
    outs = [torch.empty_like(out) for _ in range(world)]
    lses = [torch.empty_like(lse) for _ in range(world)]
    dist.all_gather(outs, out, group=group)
    dist.all_gather(lses, lse, group=group)
    return torch.cat(outs, dim=1), torch.cat(lses, dim=2)
