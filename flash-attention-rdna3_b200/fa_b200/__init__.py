"""FlashAttention-2 for NVIDIA B200 (sm_100a): hand-written CUDA kernels behind the fa_rdna3 API."""

from ._validation import is_available, unsupported_reason
from .interface import (
    alibi_slopes,
    check_status,
    flash_attention,
    flash_attention_decode,
    flash_attention_decode_paged,
    flash_attention_varlen,
    flash_attn_func,
    flash_attn_varlen_func,
)
from .sdpa import (
    disable_flash_attention,
    disable_rdna3_flash_attention,
    enable_flash_attention,
    enable_rdna3_flash_attention,
    use_flash_attention,
    use_rdna3_flash_attention,
)

__version__ = "0.1.0"

__all__ = [
    "flash_attention",
    "flash_attention_decode",
    "flash_attention_varlen",
    "flash_attention_decode_paged",
    "flash_attn_func",
    "flash_attn_varlen_func",
    "alibi_slopes",
    "is_available",
    "unsupported_reason",
    "check_status",
    "enable_flash_attention",
    "disable_flash_attention",
    "use_flash_attention",
    "enable_rdna3_flash_attention",
    "disable_rdna3_flash_attention",
    "use_rdna3_flash_attention",
]
