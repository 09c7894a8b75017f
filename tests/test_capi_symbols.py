"""The C-ABI library loads and exports every symbol that include/fa_b200.h declares, its structs have
the layout the ctypes mirror assumes, and host-side argument checks answer without touching a GPU."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from flash_attention_turing_b200 import capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "fa_b200.h"

pytestmark = pytest.mark.skipif(not capi.LIB_PATH.exists(), reason="libfa_b200.so not built")


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"^\s*(?:const\s+char\*|int|size_t)\s+(fa_\w+)\s*\(", text, flags=re.M)))


def test_header_and_ctypes_agree_on_the_symbol_list():
    assert _declared_functions() == sorted(capi.EXPORTED_SYMBOLS)


def test_every_declared_symbol_is_exported():
    lib = capi.lib()
    for name in _declared_functions():
        assert getattr(lib, name) is not None, name
    assert lib.fa_abi_version() == 2


def test_struct_layouts_match_the_header(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "fa_b200.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(FaFwdParams), sizeof(FaBwdParams),"
        " sizeof(FaKvcacheParams), sizeof(FaCombineParams), offsetof(FaFwdParams, softmax_scale),"
        " offsetof(FaBwdParams, flags), offsetof(FaKvcacheParams, num_splits)); return 0;}\n")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-I", str(HEADER.parent), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [ctypes.sizeof(capi.FaFwdParams), ctypes.sizeof(capi.FaBwdParams), ctypes.sizeof(capi.FaKvcacheParams),
            ctypes.sizeof(capi.FaCombineParams), capi.FaFwdParams.softmax_scale.offset,
            capi.FaBwdParams.flags.offset, capi.FaKvcacheParams.num_splits.offset]
    assert got == want


def test_host_side_argument_checks_need_no_gpu():
    lib = capi.lib()
    p = capi.FaFwdParams()
    rc = lib.fa_fwd(ctypes.byref(p), None)
    assert rc == -1 and b"non-NULL" in lib.fa_last_error()
    rc = lib.fa_fwd(None, None)
    assert rc == -1
    c = capi.FaCombineParams()
    assert lib.fa_combine(ctypes.byref(c), None) == -1
    b = capi.FaBwdParams()
    assert lib.fa_bwd(ctypes.byref(b), None) == -1
    k = capi.FaKvcacheParams()
    k.d = 96
    assert lib.fa_kvcache(ctypes.byref(k), None) == -2 and b"head_dim" in lib.fa_last_error()


def test_workspace_queries():
    lib = capi.lib()
    b = capi.FaBwdParams()
    b.b, b.h, b.seqlen_q, b.d = 2, 4, 130, 64
    assert lib.fa_bwd_workspace_bytes(ctypes.byref(b)) == 2 * 2 * 4 * 256 * 4  # two fp32 statistics per padded row
    b.flags = capi.FA_BWD_SINGLE_KERNEL  # plus the fp32 dQ accumulator (heads x padded rows x d)
    assert lib.fa_bwd_workspace_bytes(ctypes.byref(b)) == 2 * 2 * 4 * 256 * 4 + 4 * (2 * 256) * 64 * 4
    k = capi.FaKvcacheParams()
    k.b, k.seqlen_q, k.h, k.h_k, k.d, k.cache_batch, k.seqlen_cache, k.num_splits = 2, 1, 8, 2, 128, 2, 4096, 4
    assert lib.fa_kvcache_num_splits(ctypes.byref(k)) == 4
    rows = 2 * 8 * 1
    assert lib.fa_kvcache_workspace_bytes(ctypes.byref(k)) == 4 * rows * 128 * 4 + 256 * ((4 * rows * 4 + 255) // 256)
    k.num_splits = 1
    assert lib.fa_kvcache_workspace_bytes(ctypes.byref(k)) == 0
