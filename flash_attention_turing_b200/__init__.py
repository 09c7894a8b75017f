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
    run (dK, dV do not).  On B200 the second is the slower one at every benchmark shape: its 64 KB of reductions
    per (key tile, Q tile) pair leave the SM through the load/store unit at about 32 bytes per clock, which costs
    more than the two recomputed products cost the tensor cores."""
    from . import _ext

    _ext.load().set_single_kernel_backward(bool(on))


def device_status(reset: bool = False) -> int:
    """Synchronise the current device and return its status word: 0 when every launch of this library completed
    normally.  Bit 0 is set when a bounded wait inside a kernel gave up (the upper bits say which); it is STICKY:
    while it is set, every later forward, backward or decode launch on the device returns without computing, so
    the outputs produced since the last zero reading must be treated as invalid.  Bit 1: a ``cache_seqlens`` entry
    exceeded the cache capacity and was clamped.  ``reset=True`` clears the word after reading it.  The reference
    has no counterpart (its launches are not error-checked, ``src/flash_fwd_launch_template.h:73-89`` of
    Cy-47/flash-attention-turing)."""
    from . import _ext

    return int(_ext.load().device_status(bool(reset)))


__all__ = [
    "set_single_kernel_backward",
    "device_status",
    "flash_attn_func",
    "flash_attn_kvpacked_func",
    "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func",
    "flash_attn_varlen_kvpacked_func",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_with_kvcache",
]
