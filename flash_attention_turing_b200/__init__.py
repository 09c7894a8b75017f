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

__all__ = [
    "flash_attn_func",
    "flash_attn_kvpacked_func",
    "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func",
    "flash_attn_varlen_kvpacked_func",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_with_kvcache",
]
