"""In-tree build of the two native artefacts of this package.

* ``libfa_b200.so``   -- the C-ABI launcher library (``include/fa_b200.h``): hand-written sm_100a
  kernels compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``; no torch dependency.
* ``_fa_b200_torch*.so`` -- the thin PyTorch binding (``csrc/torch_ext.cpp``) that mirrors the five
  functions of the reference extension (``csrc/flash_attn/flash_api.cpp:717-724`` in
  Cy-47/flash-attention-turing) and links against ``libfa_b200.so``.

Replaces the reference's ``setup.py:12-49`` (``-arch=sm_75``, CUTLASS submodule).  Both outputs
land next to this file so they travel with the source tree; nothing is installed into
site-packages.  ``python -m flash_attention_turing_b200._build`` rebuilds what is out of date.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libfa_b200.so"
EXT_NAME = "_fa_b200_torch"
EXT_PATH = PKG_DIR / f"{EXT_NAME}.so"

CUDA_SOURCES = ["common.cu", "fwd_sm100.cu", "bwd_sm100.cu", "bwd_fused_sm100.cu", "kvcache_sm100.cu", "combine.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return Path(cand)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _newer(target: Path, deps) -> bool:
    """True when target exists and is newer than every dependency."""
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, log_path: Path | None = None) -> None:
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if log_path is not None:
        log_path.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(str(c) for c in cmd))


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources for sm_100a and link ``libfa_b200.so``."""
    nvcc = _cuda_home() / "bin" / "nvcc"
    OBJ_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    jobs = []
    for src in CUDA_SOURCES:
        obj = OBJ_DIR / (src + ".o")
        if force or not _newer(obj, [CSRC / src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        _run([nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", CSRC / src, "-o", obj],
             log_path=OBJ_DIR / (src + ".ptxas.log"))
        if verbose:
            print(f"[build] compiled {src}")

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        list(pool.map(compile_one, jobs))
    objs = [OBJ_DIR / (s + ".o") for s in CUDA_SOURCES]
    if force or jobs or not _newer(LIB_PATH, objs):
        _run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-cudart", "shared"])
        if verbose:
            print(f"[build] linked {LIB_PATH.name}")
    return LIB_PATH


def build_torch_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/torch_ext.cpp`` with the host compiler against this torch install."""
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_ext.cpp"
    deps = [src, *INCLUDE.glob("*.h"), LIB_PATH]
    stamp = OBJ_DIR / "torch_ext.stamp"
    tag = f"{torch.__version__}|{sys.version_info[:2]}"
    if not force and _newer(EXT_PATH, deps) and stamp.exists() and stamp.read_text() == tag:
        return EXT_PATH
    OBJ_DIR.mkdir(exist_ok=True)
    cuda_inc = _cuda_home() / "include"
    inc = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(cuda_inc), str(INCLUDE)]
    torch_lib = cpp_extension.library_paths()[0]
    cxx11 = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
        f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}",
        *[f"-I{i}" for i in inc],
        str(src), "-o", str(EXT_PATH),
        f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
        f"-L{PKG_DIR}", "-lfa_b200",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd)
    stamp.write_text(tag)
    if verbose:
        print(f"[build] built {EXT_PATH.name}")
    return EXT_PATH


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_torch_extension(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
