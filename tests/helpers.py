"""Seeded input generators and error metrics shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

# Absolute bounds of the reference's own test suite (BWD_TOLS, test_flash_attn.py:42-49 of
# Cy-47/flash-attention-turing): max |err| <= 9e-3 and mean |err| <= 2e-4 on O, dQ, dK, dV.  They are
# stated there against an fp16 SDPA oracle; here they are applied against the stricter fp32 oracle.
MAX_ABS_TOL = 9e-3
MEAN_ABS_TOL = 2e-4
LSE_TOL = 1e-3  # absolute, the tolerance the north-star states for LSE


def randn_half(gen: torch.Generator, *shape) -> torch.Tensor:
    """fp16 N(0,1) tensor drawn on the CPU from a seeded generator."""
    return torch.randn(*shape, generator=gen, dtype=torch.float32).half()


def err_stats(got: torch.Tensor, want: torch.Tensor):
    d = (got.detach().float().cpu() - want.detach().float().cpu()).abs()
    return d.max().item() if d.numel() else 0.0, d.mean().item() if d.numel() else 0.0


def emulated_reference_kernel_error(q, k, v, scale, causal, out_ref):
    """Max |err| vs the fp32 oracle of an emulation of the REFERENCE KERNEL's rounding points
    (fp16 P before the second GEMM, fp32 accumulation, fp16 output; flash_fwd_kernel.h:578,632):
    the yardstick "the reference kernel's own error" when that kernel cannot be built here."""
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    g = h // hk
    worst = 0.0
    for i in range(b):
        qf = q[i].float().transpose(0, 1)
        kf = k[i].float().repeat_interleave(g, dim=1).transpose(0, 1)
        vf = v[i].float().repeat_interleave(g, dim=1).transpose(0, 1)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        if causal:
            keep = torch.arange(sk)[None, :] <= torch.arange(sq)[:, None] + (sk - sq)
            s = s.masked_fill(~keep, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = torch.exp(s - m)
        l = p.sum(-1, keepdim=True)
        o = torch.matmul(p.half().float(), vf) / torch.where(l > 0, l, torch.ones_like(l))
        o = o.half().float().transpose(0, 1)
        worst = max(worst, (o - out_ref[i]).abs().max().item())
    return worst


def load_golden(name: str):
    from conftest import GOLDEN

    z = np.load(GOLDEN / f"{name}.npz")
    return {key: z[key] for key in z.files}


def t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))
