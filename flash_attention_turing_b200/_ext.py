"""Loads the native artefacts built by ``_build.py``; there is no fallback.

``load()`` returns the PyTorch binding module (the counterpart of the reference's
``import flash_attn_turing as flash_attn_gpu``, ``flash_attention_interface.py:5`` in
Cy-47/flash-attention-turing).  If the shared objects are missing the import fails with an
instruction to build them -- no pure-PyTorch or CPU path stands in for the kernels.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libfa_b200.so"
EXT_NAME = "_fa_b200_torch"
EXT_PATH = PKG_DIR / f"{EXT_NAME}.so"

_module = None


class NativeLibraryMissing(ImportError):
    pass


def load():
    """Import and return the torch extension module (cached)."""
    global _module
    if _module is not None:
        return _module
    for path in (LIB_PATH, EXT_PATH):
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path.name} not found in {PKG_DIR}. Build the sm_100a kernels first: "
                "`python -m flash_attention_turing_b200._build` (needs nvcc and g++). "
                "This package has no CPU or pure-PyTorch fallback."
            )
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    full_name = f"{__package__}.{EXT_NAME}"
    loader = importlib.machinery.ExtensionFileLoader(EXT_NAME, str(EXT_PATH))
    spec = importlib.util.spec_from_file_location(EXT_NAME, str(EXT_PATH), loader=loader)
    module = importlib.util.module_from_spec(spec)
    loader.exec_module(module)
    sys.modules[full_name] = module
    _module = module
    return module
