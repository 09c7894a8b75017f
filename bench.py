#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + one backward pass of causal attention at the headline point of the metric:
B=4, S_q=S_k=8192, H=32 query / 32 KV heads, D=128, fp16, seeded N(0,1) inputs (synthetic).  With N > 1
(launched under torchrun, one rank per GPU) every rank runs the same independent (batch x head) shard
-- weak scaling, no data-path collective -- and the reported value is the aggregate over ranks.

Printed by rank 0: ONE JSON line with
  value      TFLOP/s of the K timed steps, inputs resident in HBM, C-ABI calls with preallocated outputs
  e2e        the same metric through the public API (flash_attn_func + autograd) with pinned HOST
             inputs copied in and O, dQ, dK, dV copied out every step (achieved copy rates alongside)
  roofline   the dominant kernel group of the step (backward: preprocess + dQ + dK/dV launches) against the
             measured dense-GEMM peak -- the burst figure when the timed region is shorter than a second, the
             sustained one otherwise, both fractions printed; roofline_fwd and roofline_decode give the forward
             kernel and the paged split-KV decode kernel (B=64, Hq=32, Hkv=8, D=128, L in [1024, 32768], page 256)
  parity     max / mean abs error of O, dQ, dK, dV of one (batch, head) slice of the TIMED tensors against the
             fp32 oracle, next to the error of the emulated reference kernel and the bound the tests enforce
  configs    a short pass over the other benchmark configurations (C1, C2, C3, C5 at both head sizes), and the
             opt-in single-kernel backward at the headline shape
  cpu_baseline  the fp32 CPU oracle timed on this box's host cores on a bounded sample of the same workload
  seq_sharded   (N > 1 only) the long-context configuration B1 S65536 H16 D128 on the N GPUs: head-sharded and
             sequence-sharded (all-to-all and fused peer-read merge, contiguous and zig-zag K/V chunks), forward
             and backward, with the bytes each rank exchanges and the difference to the single-GPU kernels

``--impl reference`` times the reference's attention math on the host CPU (the fp32 oracle port: the
reference's CUDA extension needs an un-vendored CUTLASS tree and its Python math does not travel with
this repository), each step a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = dict(b=4, s=8192, h=32, h_k=32, d=128, causal=True)
DECODE = dict(b=64, h=32, h_k=8, d=128, page=256, pages=16384, max_pages=129, lo=1024, hi=32768)
METRIC = "attn fwd+bwd TFLOP/s (hd128 causal, S=8k)"
WORKLOAD_NAME = "H8K: B4 S8192 H32 D128 causal, forward + backward"  # the same string in both arms
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
# DRAM bytes (read + write) per launch of the kernels at exactly the workloads above, from profiler captures
# (dram__bytes_read.sum + dram__bytes_write.sum): the backward kernels from one launch each at full size, the
# forward and the decode kernel scaled from reduced-case captures by the tensor bytes a launch touches.  They
# are constants of the workload, not measured by this script; algorithmic tensor bytes for comparison: forward
# 1078 MB, backward 3494 MB, decode 4275 MB.
NCU_TRAFFIC_BYTES = dict(fwd=0.87 * 1078e6, bwd=548.5e6 + 1336.4e6 + 1590.1e6, decode=1.002 * 4275.4e6 + 4.5e6)


def fwd_flops(b, h, sq, sk, d, causal):
    f = 4.0 * b * h * sq * sk * d
    return f * 0.5 if causal else f


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return dict(hbm_gbs=float(data["hbm_gbs"]), bf16_tflops=float(data["bf16_tflops"]),
                        bf16_tflops_sustained=float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))), "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # clocks under load only: samples close to the maximum power seen
        under = [c for c, p in zip(sm, power) if power and p >= 0.6 * max(power)] or sm
        return {"sm_mhz": statistics.median(under) if under else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def cpu_attention_sample(slices: int, threads: int, s: int, d: int, causal: bool, seed: int = 1):
    """fp32 oracle forward + backward on `slices` (batch, head) slices of the workload; returns seconds."""
    import torch
    from oracle import attention_oracle as orc

    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(seed)
    q, k, v, dout = (torch.randn(1, s, slices, d, generator=gen).half() for _ in range(4))
    t0 = time.perf_counter()
    orc.attention_forward(q, k, v, None, causal)
    orc.attention_backward(q, k, v, dout, None, causal)
    return time.perf_counter() - t0


def run_reference(args, rank: int):
    """CPU arm: the reference's fp32 attention math (oracle port) on the host cores, rank 0 only."""
    if rank != 0:
        return
    w = WORKLOAD
    threads = os.cpu_count() or 1
    slices = 1
    flops = 3.5 * fwd_flops(1, slices, w["s"], w["s"], w["d"], w["causal"])
    for _ in range(args.warmup):
        cpu_attention_sample(slices, threads, w["s"], w["d"], w["causal"])
    t0 = time.perf_counter()
    for i in range(args.steps):
        cpu_attention_sample(slices, threads, w["s"], w["d"], w["causal"], seed=2 + i)
    dt = time.perf_counter() - t0
    value = flops * args.steps / dt / 1e12
    sample = f"{slices} of {w['b'] * w['h']} (batch, head) slices per step, S={w['s']} D={w['d']} causal fwd+bwd"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME, "sample": sample,
                   "note": "CPU arm: rank 0 alone computes on the host cores at every N; no GPU is used"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_profile_case(args):
    """Reduced cases for profiler captures (a few hundred MB on the device, inputs still larger than L2):
    fwd / bwd: B2 S4096 H16 D128 causal; decode: B16 Hq32 Hkv8 D128, L ~ U[1024, 32768], 4096-page pool."""
    import torch

    from flash_attention_turing_b200 import _ext, capi

    _ext.load()
    lib = capi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device=dev).manual_seed(5)
    if args.profile == "bwd_full_size":
        # ONE launch of each backward path at the benchmark size (B4 S8192 H32 D128 causal; 2.5 GB resident): for
        # single-pass traffic counters only
        w = WORKLOAD
        b, s, h, d = w["b"], w["s"], w["h"], w["d"]
        q, k, v, dout = (torch.randn(b, s, h, d, device=dev, dtype=torch.half, generator=gen) for _ in range(4))
        o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse = torch.empty(b, h, s, device=dev, dtype=torch.float32)
        capi.check(lib.fa_fwd(ctypes.byref(capi.fwd_params(q, k, v, o, lse, d ** -0.5, True)), stream))
        for flags in (capi.FA_BWD_SINGLE_KERNEL, 0):
            bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, None, d ** -0.5, True)
            bp.flags = flags
            ws = torch.empty(lib.fa_bwd_workspace_bytes(ctypes.byref(bp)), dtype=torch.uint8, device=dev)
            bp.workspace, bp.workspace_bytes = ws.data_ptr(), ws.numel()
            capi.check(lib.fa_bwd(ctypes.byref(bp), stream))
            torch.cuda.synchronize()
    elif args.profile in ("fwd", "bwd"):
        b, s, h, d = 2, 4096, 16, 128
        q, k, v, dout = (torch.randn(b, s, h, d, device=dev, dtype=torch.half, generator=gen) for _ in range(4))
        o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse = torch.empty(b, h, s, device=dev, dtype=torch.float32)
        fp = capi.fwd_params(q, k, v, o, lse, d ** -0.5, True)
        bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, None, d ** -0.5, True)
        bp.flags = args.bwd_flags
        ws = torch.empty(lib.fa_bwd_workspace_bytes(ctypes.byref(bp)), dtype=torch.uint8, device=dev)
        bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, ws, d ** -0.5, True)
        bp.flags = args.bwd_flags
        capi.check(lib.fa_fwd(ctypes.byref(fp), stream))
        for _ in range(args.profile_iters):
            if args.profile == "fwd":
                capi.check(lib.fa_fwd(ctypes.byref(fp), stream))
            else:
                capi.check(lib.fa_bwd(ctypes.byref(bp), stream))
    else:
        bb, hq, hk, d, page, pages, max_pages = 16, 32, 8, 128, 256, 4096, 129
        gen_c = torch.Generator().manual_seed(1004)
        lens = torch.randint(1024, 32768, (bb,), generator=gen_c, dtype=torch.int32)
        perm = torch.randperm(pages, generator=gen_c).to(torch.int32)
        table = torch.zeros(bb, max_pages, dtype=torch.int32)
        off = 0
        for i in range(bb):
            n = (int(lens[i]) + 1 + page - 1) // page
            table[i, :n] = perm[off:off + n]
            off += n
        kc = torch.randn(pages, page, hk, d, device=dev, dtype=torch.half, generator=gen)
        vc = torch.randn(pages, page, hk, d, device=dev, dtype=torch.half, generator=gen)
        q1 = torch.randn(bb, 1, hq, d, device=dev, dtype=torch.half, generator=gen)
        kn = torch.randn(bb, 1, hk, d, device=dev, dtype=torch.half, generator=gen)
        vn = torch.randn(bb, 1, hk, d, device=dev, dtype=torch.half, generator=gen)
        o1 = torch.empty_like(q1)
        lse1 = torch.empty(bb, hq, 1, device=dev, dtype=torch.float32)
        kp = capi.kvcache_params(q1, kc, vc, kn, vn, o1, lse1, lens.to(dev), table.to(dev), d ** -0.5, True, 4)
        need = lib.fa_kvcache_workspace_bytes(ctypes.byref(kp))
        wsk = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        kp.workspace, kp.workspace_bytes = wsk.data_ptr(), need
        for _ in range(args.profile_iters):
            capi.check(lib.fa_kvcache(ctypes.byref(kp), stream))
        kv_bytes = float((lens.double() + 1).sum()) * 2 * hk * d * 2
        print(json.dumps({"profile": "decode", "kv_bytes_per_launch": kv_bytes}))
    torch.cuda.synchronize()
    print(json.dumps({"profile": args.profile, "device_status": lib.fa_device_status(1)}))


def c3_lengths():
    """C3: 16 sequences, lengths U[256, 4096] from a fixed seed, scaled down to at most 32768 tokens."""
    import torch

    g3 = torch.Generator().manual_seed(1003)
    lens = torch.randint(256, 4097, (16,), generator=g3)
    if int(lens.sum()) > 32768:
        lens = torch.clamp(lens * 32768 // int(lens.sum()), min=256)
    return lens


def measure_configs(ext, dev, iters=10, long_iters=3, with_decode_api=False):
    """CUDA-event timings of the benchmark configurations other than the headline one, through the torch
    binding on `dev`: C1, C2, C3, C5 (both head sizes), and the opt-in single-kernel backward at the headline
    shape.  Burst numbers (a few iterations each).  Returns {name: record}."""
    import torch

    gen = torch.Generator(device=dev).manual_seed(1)
    out = {}

    def time_ms(fn, n, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def dense(name, desc, b, s, h, hk, d, causal, with_bwd, n):
        q = torch.randn(b, s, h, d, device=dev, dtype=torch.half, generator=gen)
        k = torch.randn(b, s, hk, d, device=dev, dtype=torch.half, generator=gen)
        v = torch.randn(b, s, hk, d, device=dev, dtype=torch.half, generator=gen)
        do = torch.randn_like(q)
        scale = d ** -0.5
        o, lse = ext.fwd(q, k, v, scale, causal)
        f = fwd_flops(b, h, s, s, d, causal)
        rec = {"config": desc, "fwd_ms": time_ms(lambda: ext.fwd(q, k, v, scale, causal), n)}
        rec["fwd_tflops"] = f / rec["fwd_ms"] / 1e9
        if with_bwd:
            rec["bwd_ms"] = time_ms(lambda: ext.bwd(q, k, v, o, lse, do, scale, causal), n)
            rec["bwd_tflops"] = 2.5 * f / rec["bwd_ms"] / 1e9
        out[name] = rec
        return q, k, v, do, o, lse

    dense("C1", "fwd non-causal B2 S512 H8 D64", 2, 512, 8, 8, 64, False, False, iters)
    dense("C2", "fwd+bwd causal B4 S4096 H32 D128", 4, 4096, 32, 32, 128, True, True, iters)
    # the opt-in single-kernel backward at the headline shape, next to the default two-kernel one
    q, k, v, do, o, lse = dense("H8K", "fwd+bwd causal B4 S8192 H32 D128", 4, 8192, 32, 32, 128, True, True, iters)
    ext.set_single_kernel_backward(True)
    try:
        ms = time_ms(lambda: ext.bwd(q, k, v, o, lse, do, 128 ** -0.5, True), iters)
    finally:
        ext.set_single_kernel_backward(False)
    out["H8K"]["bwd_single_kernel_ms"] = ms
    out["H8K"]["bwd_single_kernel_tflops"] = 2.5 * fwd_flops(4, 32, 8192, 8192, 128, True) / ms / 1e9
    del q, k, v, do, o, lse
    # C3: GQA varlen
    lens = c3_lengths()
    cu = torch.tensor([0] + lens.cumsum(0).tolist(), dtype=torch.int32, device=dev)
    total, mx = int(lens.sum()), int(lens.max())
    q = torch.randn(total, 32, 128, device=dev, dtype=torch.half, generator=gen)
    k = torch.randn(total, 8, 128, device=dev, dtype=torch.half, generator=gen)
    v = torch.randn(total, 8, 128, device=dev, dtype=torch.half, generator=gen)
    do = torch.randn_like(q)
    sc = 128 ** -0.5
    o, lse = ext.varlen_fwd(q, k, v, cu, cu, mx, mx, sc, True)
    f3 = float(sum(4.0 * 32 * int(n) ** 2 * 128 * 0.5 for n in lens))
    rec = {"config": f"GQA varlen fwd+bwd causal Hq32 Hkv8 D128, 16 seqs, {total} tokens",
           "fwd_ms": time_ms(lambda: ext.varlen_fwd(q, k, v, cu, cu, mx, mx, sc, True), iters),
           "bwd_ms": time_ms(lambda: ext.varlen_bwd(q, k, v, o, lse, do, cu, cu, mx, mx, sc, True), iters)}
    rec["fwd_tflops"] = f3 / rec["fwd_ms"] / 1e9
    rec["bwd_tflops"] = 2.5 * f3 / rec["bwd_ms"] / 1e9
    out["C3"] = rec
    del q, k, v, do, o, lse
    # C5: long context, all 16 heads on one GPU
    for d in (128, 64):
        dense(f"C5_D{d}", f"fwd+bwd causal B1 S65536 H16 D{d} (all 16 heads on one GPU)", 1, 65536, 16, 16, d, True, True,
              long_iters)
    if with_decode_api:
        # C4: paged decode through the public API (includes its host-side checks)
        from flash_attention_turing_b200 import flash_attn_with_kvcache

        c = DECODE
        gen_c = torch.Generator().manual_seed(1004)
        lens4 = torch.randint(c["lo"], c["hi"], (c["b"],), generator=gen_c, dtype=torch.int32)
        perm = torch.randperm(c["pages"], generator=gen_c).to(torch.int32)
        table = torch.zeros(c["b"], c["max_pages"], dtype=torch.int32)
        off = 0
        for i in range(c["b"]):
            n = (int(lens4[i]) + 1 + c["page"] - 1) // c["page"]
            table[i, :n] = perm[off:off + n]
            off += n
        kc = torch.randn(c["pages"], c["page"], c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        vc = torch.randn(c["pages"], c["page"], c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        q1 = torch.randn(c["b"], 1, c["h"], c["d"], device=dev, dtype=torch.half, generator=gen)
        kn = torch.randn(c["b"], 1, c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        vn = torch.randn_like(kn)
        ld, td = lens4.to(dev), table.to(dev)
        kv_bytes = float((lens4.double() + 1).sum()) * 2 * c["h_k"] * c["d"] * 2
        for splits in (1, 4, 16, 0):
            ms = time_ms(lambda: flash_attn_with_kvcache(q1, kc, vc, kn, vn, cache_seqlens=ld, block_table=td, causal=True,
                                                         num_splits=splits), 20)
            out[f"C4_splits{splits}"] = {"config": f"paged decode B64 Hq32 Hkv8 D128 num_splits={splits} (public API)",
                                         "ms": ms, "kv_gbs": kv_bytes / ms / 1e6}
    return out


def run_all_configs(args):
    """`--configs`: one JSON line per benchmark configuration, timed on cuda:0."""
    import torch

    from flash_attention_turing_b200 import _ext

    ext = _ext.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    for name, rec in measure_configs(ext, dev, iters=20, long_iters=3, with_decode_api=True).items():
        print(json.dumps({"name": name, **rec}), flush=True)
    print(json.dumps({"device_status": int(ext.device_status(True))}))


def measure_parity(q, k, v, dout, o, lse, dq, dk, dv, slice_bh, causal):
    """Errors of one (batch, head) slice of the timed tensors against the fp32 oracle (the checker; runs on the
    host cores), next to the errors of the emulated reference kernel and the bounds the tests enforce."""
    sys.path.insert(0, str(ROOT / "tests"))
    import torch

    import helpers
    from oracle import attention_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)  # torchrun sets OMP_NUM_THREADS=1; the checker may use the host cores
    bi, hi = slice_bh
    g = q.shape[2] // k.shape[2]
    d = q.shape[-1]
    sl = lambda x, head: x[bi:bi + 1, :, head:head + 1].float().cpu()  # noqa: E731
    qs, ks, vs, ds = sl(q, hi).half(), sl(k, hi // g).half(), sl(v, hi // g).half(), sl(dout, hi).half()
    o_ref, lse_ref = orc.attention_forward(qs, ks, vs, None, causal)
    rq, rk, rv = orc.attention_backward(qs, ks, vs, ds, None, causal)
    em = helpers.emulate_reference_kernel(qs, ks, vs, ds, d ** -0.5, causal)
    rec = {"slice": {"batch": bi, "head": hi}, "oracle": "fp32 attention math on the host cores",
           "rule": "max <= 2 x reference kernel's + one rounding event + half an fp16 ulp; mean <= 1.25 x reference kernel's",
           "lse_max_abs_err": float((lse[bi, hi].float().cpu() - lse_ref[0, 0]).abs().max()), "lse_bound": 1e-3}
    ok = rec["lse_max_abs_err"] <= 1e-3
    pairs = [("O", sl(o, hi), o_ref, em.out), ("dQ", sl(dq, hi), rq, em.dq)]
    if g == 1:  # with GQA a KV head's gradient sums its whole group: only comparable when the group is one head
        pairs += [("dK", sl(dk, hi), rk, em.dk), ("dV", sl(dv, hi), rv, em.dv)]
    n0 = len(helpers.PARITY_LOG)
    for name, got, want, emu in pairs:
        try:
            helpers.assert_within_twice_reference_kernel(name, got, want, emu)
            passed = True
        except AssertionError:
            passed = False
        r = helpers.PARITY_LOG[n0]
        n0 = len(helpers.PARITY_LOG)
        rec[name] = {"max_abs_err": r["err"], "reference_kernel_max_abs_err": r["ref"], "max_bound": r["max_bound"],
                     "mean_abs_err": r["mean"], "reference_kernel_mean_abs_err": r["refmean"],
                     "mean_bound": r["mean_bound"], "within_bounds": passed}
        ok = ok and passed
    rec["all_within_bounds"] = ok
    return rec


def bind_host_memory_near_gpu(local_rank: int):
    """Best effort: prefer the NUMA node of this rank's GPU for the host buffers allocated afterwards
    (set_mempolicy(MPOL_PREFERRED) through libc; nothing outlives the process).  Returns a small record."""
    rec = {"numa_node": None, "policy": "unchanged"}
    try:
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(local_rank)],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if bus.count(":") == 2 and len(bus.split(":")[0]) == 8:
            bus = bus[4:]  # 00000000:1b:00.0 -> 0000:1b:00.0
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text().strip())
        rec["numa_node"] = node
        if node < 0:
            rec["policy"] = "unchanged: the platform reports no NUMA node for the GPU"
            return rec
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        rc = libc.syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(64))  # set_mempolicy(MPOL_PREFERRED, mask, 64)
        rec["policy"] = "preferred" if rc == 0 else f"unchanged: set_mempolicy errno {ctypes.get_errno()}"
        try:
            cpus = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
            allowed = os.sched_getaffinity(0)
            want = set()
            for part in cpus.split(","):
                lo, _, hi = part.partition("-")
                want.update(range(int(lo), int(hi or lo) + 1))
            rec["cpus_allowed_on_node"] = len(want & allowed)
            if want & allowed:
                os.sched_setaffinity(0, want & allowed)
        except (OSError, ValueError):
            pass
    except Exception as exc:  # noqa: BLE001
        rec["policy"] = f"unchanged: {type(exc).__name__}: {exc}"[:200]
    return rec


def measure_seq_sharded(ext, dev, rank, world, iters=3):
    """The long-context configuration C5 (B1 S65536 H16 D128 causal) on the `world` GPUs of this job:
    head-sharded forward + backward (16 / world heads per rank, no communication) and sequence-sharded forward
    + backward -- K/V split over the ranks in contiguous ranges or zig-zag chunk pairs, partial (O, LSE) merged and
    dQ shares summed after an all_to_all_single (NCCL) or by ONE kernel that reads the peers' buffers over NVLink.
    Times are CUDA events, max over ranks.  Returns a dict (identical on every rank)."""
    import torch
    import torch.distributed as dist

    from flash_attention_turing_b200 import seq_parallel as sp

    s, h, d = 65536, 16, 128
    scale = d ** -0.5
    f_fwd = fwd_flops(1, h, s, s, d, True)

    def timed(fn, n=iters, warm=1):
        for _ in range(warm):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        x = torch.tensor([e0.elapsed_time(e1) / n], device=dev, dtype=torch.float64)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    def maxall(v):
        x = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    rec = {"workload": "C5: B1 S65536 H16 D128 causal", "n_gpus": world, "iters": iters}
    gen = torch.Generator(device=dev).manual_seed(1005)  # the same data on every rank
    q, k, v, do = (torch.randn(1, s, h, d, device=dev, dtype=torch.half, generator=gen) for _ in range(4))
    # (1) heads sharded: rank r takes heads [r * hl, (r + 1) * hl)
    hl = max(1, h // world)
    hs = slice((rank * hl) % h, (rank * hl) % h + hl)
    qh, kh, vh, doh = (x[:, :, hs].contiguous() for x in (q, k, v, do))
    oh, lh = ext.fwd(qh, kh, vh, scale, True)
    fwd_ms = timed(lambda: ext.fwd(qh, kh, vh, scale, True))
    bwd_ms = timed(lambda: ext.bwd(qh, kh, vh, oh, lh, doh, scale, True))
    dqh, _, _ = ext.bwd(qh, kh, vh, oh, lh, doh, scale, True)
    share = hl * world / h
    rec["head_sharded"] = {"heads_per_gpu": hl, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "fwd_tflops": f_fwd * share / fwd_ms / 1e9,
                           "bwd_tflops": 2.5 * f_fwd * share / bwd_ms / 1e9, "bytes_exchanged_per_rank": 0}
    # reference values for the sequence-sharded results: this rank's heads, computed by the single-GPU kernels
    sl = s // world
    rows = slice(rank * sl, (rank + 1) * sl)
    peer_ok = {}
    for layout in ("contiguous", "zigzag"):
        ks, vs = sp.shard_kv(k, rank, world, layout), sp.shard_kv(v, rank, world, layout)
        ent = {}
        # forward, merge after an all-to-all
        out, lse = sp.sequence_parallel_forward(q, ks, vs, scale, True, layout=layout)
        ent["fwd_all_to_all_ms"] = timed(lambda: sp.sequence_parallel_forward(q, ks, vs, scale, True, layout=layout))
        ent["fwd_max_abs_diff_vs_one_gpu"] = maxall((out[:, :, hs].float() - oh[:, rows].float()).abs().max().item())
        ent["lse_max_abs_diff_vs_one_gpu"] = maxall((lse[:, hs] - lh[:, :, rows]).abs().max().item())
        # bytes one rank sends (= receives): its partial O for the other ranks' row slices + LSE
        ent["fwd_bytes_exchanged_per_rank"] = int((world - 1) / world * (s * h * d * 2 + s * h * 4))
        out_all, lse_all = sp.sequence_parallel_forward(q, ks, vs, scale, True, gather_output=True, layout=layout)
        dq, _, _ = sp.sequence_parallel_backward(q, ks, vs, out_all, lse_all, do, scale, True, layout=layout)
        ent["bwd_all_to_all_ms"] = timed(lambda: sp.sequence_parallel_backward(q, ks, vs, out_all, lse_all, do, scale, True,
                                                                                layout=layout))
        ent["dq_max_abs_diff_vs_one_gpu"] = maxall((dq[:, :, hs].float() - dqh[:, rows].float()).abs().max().item())
        ent["bwd_bytes_exchanged_per_rank"] = int((world - 1) / world * s * h * d * 2)
        # the same with the exchange fused into the merge kernel (peer reads over NVLink)
        if layout not in peer_ok:
            peer_ok[layout] = sp.peer_memory_available_for(q, layout)
        if peer_ok[layout]:
            # with zig-zag K/V chunks the rank also produces zig-zag ROWS (chunks r and 2*world-1-r): under the
            # causal mask that gives every rank the same number of parts to fetch and merge
            rl = layout
            want_o = sp.gather_owned_rows(out_all, rank, world, rl)
            dq_all = [torch.empty_like(dq) for _ in range(world)]
            dist.all_gather(dq_all, dq)
            want_dq = sp.gather_owned_rows(torch.cat(dq_all, dim=1), rank, world, rl)
            del dq_all
            o_p, l_p = sp.sequence_parallel_forward_p2p(q, ks, vs, scale, True, layout=layout, row_layout=rl)
            ent["fwd_peer_read_ms"] = timed(lambda: sp.sequence_parallel_forward_p2p(q, ks, vs, scale, True, layout=layout,
                                                                                      row_layout=rl))
            ent["fwd_peer_read_max_abs_diff_vs_all_to_all"] = maxall((o_p.float() - want_o.float()).abs().max().item())
            dq_p, _, _ = sp.sequence_parallel_backward_p2p(q, ks, vs, out_all, lse_all, do, scale, True, layout=layout,
                                                           row_layout=rl)
            ent["bwd_peer_read_ms"] = timed(lambda: sp.sequence_parallel_backward_p2p(q, ks, vs, out_all, lse_all, do, scale,
                                                                                       True, layout=layout, row_layout=rl))
            ent["dq_peer_read_max_abs_diff_vs_all_to_all"] = maxall((dq_p.float() - want_dq.float()).abs().max().item())
            ent["peer_read_rows"] = rl
            del want_o, want_dq
            ent["peer_read"] = "symmetric memory, plain loads over NVLink"
        else:
            ent["peer_read"] = "unavailable: " + (sp.last_peer_memory_error() or "a peer could not map the buffers")[:200]
        # the local kernels alone (no exchange): what is left is the exchange + merge
        nch = 2 if layout == "zigzag" else 1
        ob = torch.empty((nch, 1, s, h, d), dtype=q.dtype, device=dev)
        lb = torch.empty((nch, 1, h, s), dtype=torch.float32, device=dev)
        ent["fwd_local_kernels_ms"] = timed(lambda: sp.rank_partials_inplace(q, ks, vs, rank, world, scale, True, layout, ob, lb))
        dkb, dvb = torch.empty_like(ks), torch.empty_like(vs)
        ent["bwd_local_kernels_ms"] = timed(lambda: sp.rank_backward_inplace(q, ks, vs, out_all, lse_all, do, rank, world, scale,
                                                                             True, layout, ob, dkb, dvb))
        for key in ("fwd_all_to_all_ms", "fwd_peer_read_ms"):
            if key in ent:
                ent[key.replace("_ms", "_tflops")] = f_fwd / ent[key] / 1e9
        for key in ("bwd_all_to_all_ms", "bwd_peer_read_ms"):
            if key in ent:
                ent[key.replace("_ms", "_tflops")] = 2.5 * f_fwd / ent[key] / 1e9
        best_fwd = min(ent.get("fwd_peer_read_ms", 1e30), ent["fwd_all_to_all_ms"])
        ent["fwd_best_over_head_sharded"] = best_fwd / fwd_ms
        ent["fwd_exchange_and_merge_ms"] = max(0.0, best_fwd - ent["fwd_local_kernels_ms"])  # what is left beside the kernels
        if ent["fwd_exchange_and_merge_ms"] > 0.05:
            ent["fwd_exchange_gbs_per_rank"] = ent["fwd_bytes_exchanged_per_rank"] / ent["fwd_exchange_and_merge_ms"] / 1e6
        ent["what_is_left"] = ("the exchange of the partial O (fwd_bytes_exchanged_per_rank over NVLink; measured peer copy rate "
                               "770 GB/s per direction) and the merge kernel run AFTER the local kernels: nothing overlaps them")
        rec[layout] = ent
        del out, lse, out_all, lse_all, dq, ob, lb, dkb, dvb
    return rec


def run_sharded(args):
    """`--sharded` (under torchrun): only the long-context multi-GPU measurement, one JSON line."""
    import torch
    import torch.distributed as dist

    from flash_attention_turing_b200 import _ext

    ext = _ext.load()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    rec = measure_seq_sharded(ext, dev, rank, world)
    rec["device_status"] = int(ext.device_status(True))
    if rank == 0:
        print(json.dumps(rec), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--skip-decode", action="store_true", help="skip the paged-decode measurement (needs 18 GB)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-parity", action="store_true")
    ap.add_argument("--skip-configs", action="store_true")
    ap.add_argument("--skip-seq-sharded", action="store_true")
    ap.add_argument("--profile", choices=["fwd", "bwd", "decode", "bwd_full_size"], default=None,
                    help="run a few launches of one kernel group on a reduced case and exit (for ncu captures)")
    ap.add_argument("--profile-iters", type=int, default=3)
    ap.add_argument("--bwd-flags", type=int, default=0,
                    help="flags of FaBwdParams for --profile bwd (1 = FA_BWD_SINGLE_KERNEL)")
    ap.add_argument("--sharded", action="store_true",
                    help="multi-GPU runs of the long-context config (B1 S65536 H16 D128 causal): head-sharded forward + "
                         "backward (no communication) and the sequence-sharded forward with its (O, LSE) merge")
    ap.add_argument("--configs", action="store_true",
                    help="time the five benchmark configs (C1..C5) through the torch binding on one GPU and exit")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args)
        return
    if args.configs:
        run_all_configs(args)
        return
    if args.sharded:
        run_sharded(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    from flash_attention_turing_b200 import _ext, capi, flash_attn_func

    ext = _ext.load()  # raises when the native library is missing: there is no fallback to measure
    lib = capi.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU for --impl ours"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # the sequence-sharded part reads peer memory with plain loads
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_src = load_peaks()
    numa = bind_host_memory_near_gpu(local_rank)  # before any pinned host buffer is allocated

    w = WORKLOAD
    b, s, h, hk, d, causal = w["b"], w["s"], w["h"], w["h_k"], w["d"], w["causal"]
    scale = d ** -0.5
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    q, k, v, dout = (torch.randn(b, s, n, d, device=dev, dtype=torch.half, generator=gen) for n in (h, hk, hk, h))
    o = torch.empty_like(q)
    lse = torch.empty(b, h, s, device=dev, dtype=torch.float32)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fp = capi.fwd_params(q, k, v, o, lse, scale, causal)
    bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, None, scale, causal)
    ws = torch.empty(lib.fa_bwd_workspace_bytes(ctypes.byref(bp)), dtype=torch.uint8, device=dev)
    bp = capi.bwd_params(q, k, v, o, dout, lse, dq, dk, dv, ws, scale, causal)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    f_fwd = fwd_flops(b, h, s, s, d, causal)
    f_bwd = 2.5 * f_fwd

    def step():
        capi.check(lib.fa_fwd(ctypes.byref(fp), stream))
        capi.check(lib.fa_bwd(ctypes.byref(bp), stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        x = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    def timed(fn, iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- main timed region: W warm-up steps, then exactly K steps ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # runs through the warm-up, the timed region and the per-kernel timing loops
    for _ in range(args.warmup):
        step()
    total_ms = timed(step, args.steps)
    ms_per_step = total_ms / args.steps
    value = (f_fwd + f_bwd) * world / (ms_per_step * 1e-3) / 1e12
    status = lib.fa_device_status(1)

    # ---- per-kernel durations (same inputs, after the main region) ----
    reps = max(5, min(args.steps, 20))
    fwd_ms = timed(lambda: capi.check(lib.fa_fwd(ctypes.byref(fp), stream)), reps) / reps
    pre_ms = timed(lambda: capi.check(lib.fa_bwd_stages(ctypes.byref(bp), 1, stream)), reps) / reps
    dq_ms = timed(lambda: capi.check(lib.fa_bwd_stages(ctypes.byref(bp), 2, stream)), reps) / reps
    dkdv_ms = timed(lambda: capi.check(lib.fa_bwd_stages(ctypes.byref(bp), 4, stream)), reps) / reps
    bwd_ms = pre_ms + dq_ms + dkdv_ms
    clocks = sampler.stop() if rank == 0 else None
    # denominator: the burst GEMM figure when the timed region is shorter than a second (the clocks have not
    # settled under the power cap yet), the sustained one otherwise; both fractions are printed
    burst_regime = args.steps * ms_per_step < 1000.0
    tensor_peak = peaks["bf16_tflops"] if burst_regime else peaks["bf16_tflops_sustained"]

    def tensor_roofline(flops, ms, kernel, traffic):
        ach = flops / (ms * 1e-3) / 1e12
        return {"kernel": kernel, "bound": "tensor", "achieved": ach, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": ach / tensor_peak, "frac_burst": ach / peaks["bf16_tflops"],
                "frac_sustained": ach / peaks["bf16_tflops_sustained"], "frac_of_nominal_2250": ach / 2250.0,
                "traffic": traffic,
                "peak_source": f"{peak_src} (cuBLAS bf16 " + ("burst" if burst_regime else "sustained") +
                               f": timed region {args.steps * ms_per_step / 1e3:.2f} s)", "ms_per_launch": ms}

    roofline = tensor_roofline(f_bwd, bwd_ms, "backward: bwd_preprocess + bwd_dq_kernel + bwd_dkdv_kernel (2.5x forward FLOPs)",
                               NCU_TRAFFIC_BYTES["bwd"])
    roofline["ms_by_kernel"] = {"bwd_preprocess_kernel": pre_ms, "bwd_dq_kernel": dq_ms, "bwd_dkdv_kernel": dkdv_ms}
    roofline_fwd = tensor_roofline(f_fwd, fwd_ms, "fwd_kernel<128>", NCU_TRAFFIC_BYTES["fwd"])

    # ---- parity of the timed tensors (rank 0): one (batch, head) slice against the oracle ----
    parity = None
    if rank == 0 and not args.skip_parity:
        step()
        torch.cuda.synchronize()
        parity = measure_parity(q, k, v, dout, o, lse, dq, dk, dv, (b - 1, 5 % h), causal)

    # ---- end to end through the public API, host buffers in and out every step ----
    hq, hk_, hv, hdo = (x.cpu().pin_memory() for x in (q, k, v, dout))
    ho, hdq, hdk, hdv = (torch.empty_like(x, device="cpu").pin_memory() for x in (q, q, k, v))

    def e2e_step():
        qd = hq.to(dev, non_blocking=True).requires_grad_(True)
        kd = hk_.to(dev, non_blocking=True).requires_grad_(True)
        vd = hv.to(dev, non_blocking=True).requires_grad_(True)
        dd = hdo.to(dev, non_blocking=True)
        out = flash_attn_func(qd, kd, vd, causal=causal)
        gq, gk, gv = torch.autograd.grad(out, (qd, kd, vd), dd)
        ho.copy_(out.detach(), non_blocking=True)
        hdq.copy_(gq, non_blocking=True)
        hdk.copy_(gk, non_blocking=True)
        hdv.copy_(gv, non_blocking=True)

    # The same steps as a three-stage pipeline, as a host that feeds the operator from host memory would run
    # them: copy-in of step i+1, the kernels of step i and copy-out of step i-1 overlap on three streams
    # (PCIe is full duplex).  Every step still copies its own inputs in and its own results out inside the
    # timed region; device input buffers are double-buffered, ordering is by events.
    s_in, s_c, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    dbuf = [[torch.empty_like(x) for x in (q, k, v, dout)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_pipeline(n):
        main = torch.cuda.current_stream()
        for st in (s_in, s_c, s_out):
            st.wait_stream(main)
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_free[b])  # the kernels of step i-2 have read this buffer set
                for dst, src in zip(dbuf[b], (hq, hk_, hv, hdo)):
                    dst.copy_(src, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[b])
                qd, kd, vd = (x.detach().requires_grad_(True) for x in dbuf[b][:3])
                out = flash_attn_func(qd, kd, vd, causal=causal)
                grads = torch.autograd.grad(out, (qd, kd, vd), dbuf[b][3])
                ev_free[b].record(s_c)
                ev_done[b].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                for dst, src in zip((ho, hdq, hdk, hdv), (out.detach(),) + tuple(grads)):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
        for st in (s_in, s_c, s_out):
            main.wait_stream(st)

    # The pipeline is timed over the K steps of the run (at most 50): its first copy-in and last copy-out have
    # nothing to overlap with, which costs about one and a half steps however many steps follow.
    e2e_steps = max(3, min(args.steps, 50))
    seq_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_seq_ms = timed(e2e_step, seq_steps) / seq_steps
    e2e_pipeline(3)
    e2e_ms = timed(lambda: e2e_pipeline(e2e_steps), 1) / e2e_steps
    e2e_value = (f_fwd + f_bwd) * world / (e2e_ms * 1e-3) / 1e12
    h2d = sum(x.numel() * 2 for x in (q, k, v, dout))
    d2h = sum(x.numel() * 2 for x in (q, q, k, v))

    # the copies alone, both directions at once (what bounds the pipelined step), slowest rank
    def copies_only():
        with torch.cuda.stream(s_in):
            for dst, src in zip(dbuf[0], (hq, hk_, hv, hdo)):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            for dst, src in zip((ho, hdq, hdk, hdv), dbuf[1]):
                dst.copy_(src, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)

    copies_only()
    copy_ms = timed(copies_only, 3) / 3
    copy_rates = {"h2d_gbs_per_rank": h2d / copy_ms / 1e6, "d2h_gbs_per_rank": d2h / copy_ms / 1e6,
                  "ms_both_directions": copy_ms, "host_memory": numa}
    del hq, hk_, hv, hdo, ho, hdq, hdk, hdv, dbuf

    # ---- paged split-KV decode (HBM-bound), kernel path through the C ABI ----
    decode = None
    roofline_decode = None
    del q, k, v, dout, o, dq, dk, dv, ws
    torch.cuda.empty_cache()
    if not args.skip_decode:
        c = DECODE
        gen_c = torch.Generator().manual_seed(1004)
        lens = torch.randint(c["lo"], c["hi"], (c["b"],), generator=gen_c, dtype=torch.int32)
        perm = torch.randperm(c["pages"], generator=gen_c).to(torch.int32)
        table = torch.zeros(c["b"], c["max_pages"], dtype=torch.int32)
        off = 0
        for i in range(c["b"]):
            n = (int(lens[i]) + 1 + c["page"] - 1) // c["page"]
            table[i, :n] = perm[off:off + n]
            off += n
        kc = torch.randn(c["pages"], c["page"], c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        vc = torch.randn(c["pages"], c["page"], c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        q1 = torch.randn(c["b"], 1, c["h"], c["d"], device=dev, dtype=torch.half, generator=gen)
        kn = torch.randn(c["b"], 1, c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        vn = torch.randn(c["b"], 1, c["h_k"], c["d"], device=dev, dtype=torch.half, generator=gen)
        o1 = torch.empty_like(q1)
        lse1 = torch.empty(c["b"], c["h"], 1, device=dev, dtype=torch.float32)
        lens_d, table_d = lens.to(dev), table.to(dev)
        kv_bytes = float((lens.double() + 1).sum()) * 2 * c["h_k"] * c["d"] * 2
        alg_bytes = (kv_bytes + 2 * c["b"] * c["h"] * c["d"] * 2 + 2 * 2 * c["b"] * c["h_k"] * c["d"] * 2 +
                     4 * (c["b"] + float(((lens + 1 + c["page"] - 1) // c["page"]).sum())) + 4 * c["b"] * c["h"])
        decode = {"metric": "paged split-KV decode HBM GB/s", "unit": "GB/s", "algorithmic_bytes": alg_bytes,
                  "config": "B64 Hq32 Hkv8 D128 L~U[1024,32768] page256 pool 16384 pages", "by_num_splits": {}}
        best = None
        for splits in (1, 4, 16, 0):
            kp = capi.kvcache_params(q1, kc, vc, kn, vn, o1, lse1, lens_d, table_d, c["d"] ** -0.5, True, splits)
            need = lib.fa_kvcache_workspace_bytes(ctypes.byref(kp))
            wsk = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
            kp.workspace, kp.workspace_bytes = wsk.data_ptr(), need
            fn = lambda: capi.check(lib.fa_kvcache(ctypes.byref(kp), stream))  # noqa: E731
            for _ in range(3):
                fn()
            ms = timed(fn, 20) / 20
            gbs = alg_bytes * world / (ms * 1e-3) / 1e9
            decode["by_num_splits"][str(splits)] = {"ms": ms, "gbs": gbs,
                                                    "effective_splits": lib.fa_kvcache_num_splits(ctypes.byref(kp))}
            if best is None or gbs > best[1]:
                best = (splits, gbs, ms)
        decode["value"] = best[1]
        per_gpu = best[1] / world
        roofline_decode = {"kernel": "decode_kernel<128> + combine_kernel<128> + append_kernel", "bound": "hbm",
                           "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
                           "frac_of_nominal_8000": per_gpu / 8000.0, "traffic": NCU_TRAFFIC_BYTES["decode"], "num_splits": best[0],
                           "peak_source": f"{peak_src} (copy bandwidth)", "ms_per_launch": best[2]}
        status |= lib.fa_device_status(1)
        del kc, vc

    # ---- the other benchmark configurations, a short pass each (rank 0's GPU; the other ranks wait) ----
    configs = None
    if not args.skip_configs:
        torch.cuda.empty_cache()
        if rank == 0:
            configs = measure_configs(ext, dev, iters=5, long_iters=2)
            status |= lib.fa_device_status(1)
        barrier()

    # ---- N > 1: the long-context configuration sharded by head and by sequence over the N GPUs ----
    seq_sharded = None
    if world > 1 and not args.skip_seq_sharded:
        torch.cuda.empty_cache()
        try:
            seq_sharded = measure_seq_sharded(ext, dev, rank, world)
        except Exception as exc:  # noqa: BLE001  recorded, never silently dropped
            seq_sharded = {"error": f"{type(exc).__name__}: {exc}"[:400]}
        status |= lib.fa_device_status(1)

    # ---- CPU baseline: fp32 oracle on the host cores, bounded sample, rank 0 only ----
    cpu_baseline = None
    if rank == 0 and not args.skip_cpu_baseline:
        threads = os.cpu_count() or 1
        slices = 4
        cpu_attention_sample(1, threads, 2048, d, causal)  # warm the thread pool
        sec = cpu_attention_sample(slices, threads, s, d, causal)
        reps_cpu = 1
        while sec < 10.0 and reps_cpu < 6:
            sec += cpu_attention_sample(slices, threads, s, d, causal, seed=10 + reps_cpu)
            reps_cpu += 1
        cpu_flops = 3.5 * fwd_flops(1, slices, s, s, d, causal) * reps_cpu
        cpu_baseline = {"value": cpu_flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{slices * reps_cpu} of {b * h} (batch, head) slices of the workload "
                                  f"(S={s}, D={d}, causal, fwd+bwd), fp32 torch oracle, {sec:.1f} s"}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "per_gpu": "one such workload per GPU (Hq = Hkv = 32)",
                       "sharding": "independent (batch x head) shards per GPU, no collective",
                       "l2": "inputs_larger_than_l2 (q,k,v,dO,O = 5 x 268 MB vs 126 MB L2)"},
            "fwd_tflops": f_fwd / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": f_bwd / (bwd_ms * 1e-3) / 1e12,
            "roofline": roofline, "roofline_fwd": roofline_fwd, "roofline_decode": roofline_decode,
            "decode": decode, "cpu_baseline": cpu_baseline, "parity": parity, "configs": configs,
            "seq_sharded": seq_sharded,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "path": "flash_attn_func + torch.autograd.grad, pinned host q,k,v,dO in; O,dQ,dK,dV out; "
                            "copy-in, kernels and copy-out of consecutive steps overlap on three streams",
                    "ms_per_step_unpipelined": e2e_seq_ms,
                    "value_unpipelined": (f_fwd + f_bwd) * world / (e2e_seq_ms * 1e-3) / 1e12,
                    "copies_alone": copy_rates,
                    "bound": "host <-> device copies (PCIe, full duplex): the step cannot be shorter than "
                             "copies_alone.ms_both_directions"},
            "gpu_launches": 4 * args.steps, "clocks": clocks, "device_status": status,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
