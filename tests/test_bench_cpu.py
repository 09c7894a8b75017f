"""The reference arm of bench.py runs on the host cores alone; its JSON line is checked here against the
benchmark contract (the GPU arm is exercised on the GPU box)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                          capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["unit"] == "TFLOP/s" and rec["higher_is_better"] is True
    assert rec["metric"] == "attn fwd+bwd TFLOP/s (hd128 causal, S=8k)"
    assert rec["steps"] == 1 and rec["warmup"] == 0 and rec["value"] > 0 and rec["ms_per_step"] > 0
    assert rec["config"]["workload"].startswith("H8K: B4 S8192 H32 D128 causal")
    assert rec["cpu_baseline"]["kind"] == "port" and rec["cpu_baseline"]["cores"] >= 1
    assert rec["cpu_baseline"]["value"] == rec["value"] == rec["e2e"]["value"]
    assert rec["e2e"]["h2d_bytes_per_step"] == 0 and rec["e2e"]["d2h_bytes_per_step"] == 0
    assert rec["vs_baseline"] is None


def test_other_ranks_of_the_reference_arm_exit_without_work():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                           "--warmup", "0"], capture_output=True, text=True, timeout=120, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert not [l for l in proc.stdout.splitlines() if l.startswith("{")]
