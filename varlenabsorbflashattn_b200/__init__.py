"""B200-native packed variable-length attention and absorbed target attention.

Public surface (same names and signatures as the reference packages):
    packed_varlen_attn, set_validate_cu_seqlens            (triton_fa_varlen_v2)
    packed_target_attn, target_attn_inner, prepare_target_attn_indices   (triton_target_attn_absorb)
All compute is in the in-tree CUDA library libvafa_b200.so (C ABI: include/vafa.h).
"""
from .varlen import (packed_varlen_attn, packed_varlen_attn_with_lse, set_validate_cu_seqlens, set_impl,
                     set_backward_mode)
from .absorb import packed_target_attn, target_attn_inner, prepare_target_attn_indices

__all__ = [
    "packed_varlen_attn", "packed_varlen_attn_with_lse", "set_validate_cu_seqlens", "set_impl", "set_backward_mode",
    "packed_target_attn", "target_attn_inner", "prepare_target_attn_indices",
]
