"""B200 (sm_100a) FlashAttention behind the operator API of Cy-47/flash-attention-turing.

``from flash_attention_turing_b200 import flash_attn_func`` replaces
``from flash_attention_interface import flash_attn_func`` of the reference.  The native library is
loaded on first use; importing this package needs neither a GPU nor the built shared objects.
"""
from .flash_attention_interface import (  # noqa: F401
    flash_attn_func,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache,
)



def set_single_kernel_backward(on: bool) -> None:
    """Select the backward path of every ``flash_attn_*`` function of this process.

    ``False`` (default): a dQ kernel and a dK/dV kernel (seven products, like the two kernels of the reference,
    ``csrc/flash_attn/src/flash_bwd_launch_template.h:84-138`` of Cy-47/flash-attention-turing); every gradient
    is bitwise reproducible.  ``True``: one kernel with the five algorithmic products; dQ is accumulated with
    global fp32 reductions whose order depends on scheduling, so dQ may differ in the last bits from run to
    run (dK, dV do not).  On B200 the second is the slower one at every benchmark shape: its reductions load
    the L2 cache more than the recomputed products load the tensor cores."""
    from . import _ext

    _ext.load().set_single_kernel_backward(bool(on))


__all__ = [
    "set_single_kernel_backward",
    "flash_attn_func",
    "flash_attn_kvpacked_func",
    "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func",
    "flash_attn_varlen_kvpacked_func",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_with_kvcache",
]
