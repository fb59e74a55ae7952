"""Drop-in ``torch.nn.functional.scaled_dot_product_attention`` hook.

``enable_flash_attention()`` swaps ``F.scaled_dot_product_attention`` for a dispatcher that sends the calls
the kernels support to :func:`flash_attention` / :func:`flash_attention_decode` and everything else to the
original function. Behaviour follows fa_rdna3/sdpa.py of the reference (routing rules :116-150, patching
:153-199); the reference's function names are kept as aliases so existing callers keep working.
"""
from contextlib import contextmanager
import math
from numbers import Real
import threading

import torch
import torch.nn.functional as F

from ._validation import is_available
from .interface import flash_attention, flash_attention_decode, _SUPPORTED_HEAD_DIMS

_original_sdpa = None
_patch_lock = threading.RLock()
_context_depth = 0
_context_installed = False
_dispatch_bypass_state = threading.local()

# A query of at most this many rows against at least this many keys goes to split-K decode, which
# spreads the cache over the whole GPU instead of one CTA pair per (batch, head).
_DECODE_MAX_QUERY = 8
_DECODE_MIN_KEY = 1024

# With gradients enabled and both sequences this short, launch overhead of the separate backward
# kernels dominates and the stock fused math backward is left in charge.
_MIN_TRAIN_SEQLEN = 16


def _is_tiny_fp32_inference(query, key, value, attn_mask, is_causal, requires_backward):
    return (
        not requires_backward
        and not is_causal
        and query.dtype == torch.float32
        and query.shape[-1] == 128
        and query.shape == key.shape == value.shape
        and query.shape[-2] <= 32
        and (attn_mask is None or attn_mask.dtype == torch.float32)
    )


def _is_supported_mask(attn_mask, query, key):
    if attn_mask is None:
        return True
    if not isinstance(attn_mask, torch.Tensor):
        return False
    if attn_mask.device != query.device or attn_mask.requires_grad:
        return False
    if attn_mask.dtype not in (torch.bool, query.dtype, torch.float32):
        return False
    target = (query.shape[0], query.shape[1], query.shape[2], key.shape[2])
    try:
        return torch.broadcast_shapes(tuple(attn_mask.shape), target) == target
    except RuntimeError:
        return False


def _is_supported_scale(scale):
    if scale is None:
        return True
    return not isinstance(scale, bool) and isinstance(scale, Real) and math.isfinite(float(scale))


def _is_supported(query, key, value, attn_mask, dropout_p, enable_gqa, scale):
    """True when the call can be served by the kernels (fa_rdna3/sdpa.py:72-105)."""
    if not all(isinstance(t, torch.Tensor) for t in (query, key, value)):
        return False
    if not query.is_cuda or not is_available(query.device):
        return False
    if key.device != query.device or value.device != query.device:
        return False
    if query.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        return False
    if key.dtype != query.dtype or value.dtype != query.dtype:
        return False
    if not (query.dim() == key.dim() == value.dim() == 4):
        return False
    if not (query.shape[0] == key.shape[0] == value.shape[0]):
        return False
    head_dim = query.shape[-1]
    if not (0 < head_dim <= 512) or key.shape[-1] != head_dim or value.shape[-1] != head_dim:
        return False  # head dims that are not a power of two are padded inside flash_attention
    if query.shape[-2] <= 0 or key.shape[-2] <= 0 or key.shape[-2] != value.shape[-2]:
        return False
    hq, hk = query.shape[-3], key.shape[-3]
    if hq <= 0 or hk <= 0 or hk != value.shape[-3]:
        return False
    if hq != hk and not (enable_gqa and hq % hk == 0):
        return False
    if not _is_supported_mask(attn_mask, query, key) or not _is_supported_scale(scale):
        return False
    if isinstance(dropout_p, bool) or not isinstance(dropout_p, Real) or dropout_p != 0.0:
        return False
    return True


def _mask_to_bias(attn_mask):
    """Boolean masks become an fp32 0 / -inf additive bias; float masks pass through."""
    if attn_mask is None:
        return None
    if attn_mask.dtype == torch.bool:
        return torch.zeros_like(attn_mask, dtype=torch.float32).masked_fill(~attn_mask, float("-inf"))
    return attn_mask


def _call_original(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa):
    return _original_sdpa(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p,
                          is_causal=is_causal, scale=scale, enable_gqa=enable_gqa)


def _dispatch_sdpa(query, key, value, attn_mask=None, dropout_p=0.0,
                   is_causal=False, scale=None, enable_gqa=False):
    if getattr(_dispatch_bypass_state, "depth", 0):
        if _original_sdpa is None:
            raise RuntimeError("SDPA bypass requires an installed dispatcher")
        return _call_original(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa)
    # The kernels' causal mask is bottom-right aligned while SDPA's is top-left, so causal calls are
    # only taken when both agree: square shapes and no extra mask.
    causal_ok = not is_causal or (attn_mask is None and query.shape[-2] == key.shape[-2])
    if not (_is_supported(query, key, value, attn_mask, dropout_p, enable_gqa, scale) and causal_ok):
        return _call_original(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa)

    requires_backward = torch.is_grad_enabled() and (
        query.requires_grad or key.requires_grad or value.requires_grad)
    if (_is_tiny_fp32_inference(query, key, value, attn_mask, is_causal, requires_backward)
            and torch.compiler.is_compiling()):
        for t in (query, key, value):
            torch._dynamo.mark_static(t, 2)
        return flash_attention(query, key, value, softmax_scale=scale, bias=_mask_to_bias(attn_mask))
    if requires_backward and query.shape[-2] <= _MIN_TRAIN_SEQLEN and key.shape[-2] <= _MIN_TRAIN_SEQLEN:
        return _call_original(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa)
    bias = _mask_to_bias(attn_mask)
    if (bias is None and not is_causal and not requires_backward
            and query.dtype in (torch.float16, torch.bfloat16)
            and query.shape[-1] in _SUPPORTED_HEAD_DIMS
            and query.shape[-2] <= _DECODE_MAX_QUERY
            and key.shape[-2] >= _DECODE_MIN_KEY):
        return flash_attention_decode(query, key, value, softmax_scale=scale)
    return flash_attention(query, key, value, causal=is_causal, softmax_scale=scale, bias=bias)


def enable_flash_attention():
    """Route supported ``scaled_dot_product_attention`` calls to the B200 kernels."""
    global _original_sdpa
    with _patch_lock:
        if _original_sdpa is None:
            _original_sdpa = F.scaled_dot_product_attention
        if F.scaled_dot_product_attention is _original_sdpa:
            F.scaled_dot_product_attention = _dispatch_sdpa


def disable_flash_attention():
    """Restore the original ``scaled_dot_product_attention``."""
    with _patch_lock:
        if _original_sdpa is not None and F.scaled_dot_product_attention is _dispatch_sdpa:
            F.scaled_dot_product_attention = _original_sdpa


@contextmanager
def _bypass_flash_attention():
    """Within the block (this thread only) the dispatcher forwards every call to the original."""
    depth = getattr(_dispatch_bypass_state, "depth", 0)
    _dispatch_bypass_state.depth = depth + 1
    try:
        yield
    finally:
        _dispatch_bypass_state.depth = depth


@contextmanager
def use_flash_attention():
    """Temporarily route supported SDPA calls through the B200 kernels; nests and is thread-safe."""
    global _context_depth, _context_installed
    with _patch_lock:
        if _context_depth == 0:
            already = F.scaled_dot_product_attention is _dispatch_sdpa
            enable_flash_attention()
            _context_installed = (not already) and F.scaled_dot_product_attention is _dispatch_sdpa
        _context_depth += 1
    try:
        yield
    finally:
        with _patch_lock:
            _context_depth -= 1
            if _context_depth == 0:
                if _context_installed:
                    disable_flash_attention()
                _context_installed = False


# Names used by the reference package (fa_rdna3/sdpa.py:153-199), kept so callers can switch unchanged.
enable_rdna3_flash_attention = enable_flash_attention
disable_rdna3_flash_attention = disable_flash_attention
use_rdna3_flash_attention = use_flash_attention
_bypass_rdna3_flash_attention = _bypass_flash_attention
