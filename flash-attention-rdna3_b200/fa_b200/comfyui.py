"""ComfyUI integration: an attention override for `transformer_options` and the model-patch node that installs it.

Behaviour follows fa_rdna3/comfyui.py of the reference (the adapter at :84-251, the node at :260-302):

* ComfyUI hands attention `(batch, tokens, heads * head_dim)` tensors, or `(batch, heads, tokens, head_dim)` with
  `skip_reshape`; the override brings them to the head layout, sends the call to :func:`flash_attention` when the
  dispatcher's own rules (`sdpa._is_supported`) accept it, and restores the layout the caller asked for.
* Everything else goes to ComfyUI's attention function untouched: calls that want fp32 accumulation on 16-bit inputs,
  `low_precision_attention=False`, shapes that do not split into heads, masks or scales the kernels do not take. The
  fall-back runs with the process-wide SDPA hook bypassed, so it cannot come back in through the other door.
* An override that was already installed keeps precedence: it is called with this adapter as the attention function
  it may delegate to.

Nothing here computes anything; ComfyUI itself is imported only to fetch its precision rule when the node patches a
model, so the module loads (and is tested) without ComfyUI.
"""
import logging
from functools import wraps

import torch

from ._validation import unsupported_reason
from .interface import flash_attention
from .sdpa import _bypass_flash_attention, _is_supported, _mask_to_bias, enable_flash_attention

logger = logging.getLogger(__name__)

# the keyword arguments ComfyUI's attention functions share, with their defaults
_LAYOUT_DEFAULTS = {"mask": None, "attn_precision": None, "skip_reshape": False, "skip_output_reshape": False}


def _split_heads(tensor, head_dim):
    """(batch, tokens, heads * head_dim) -> (batch, heads, tokens, head_dim), as a view."""
    batch, tokens, width = tensor.shape
    return tensor.reshape(batch, tokens, width // head_dim, head_dim).transpose(1, 2)


def _to_head_layout(query, key, value, heads, already_split, grouped):
    """(q, k, v) as (batch, heads, tokens, head_dim), or None when the call does not describe such tensors: wrong
    rank, batch sizes that differ, a width that is not a whole number of heads, or key / value head counts that are
    neither the query's nor (with `grouped`) a divisor of it."""
    if type(heads) is not int or heads <= 0:
        return None
    tensors = (query, key, value)
    if any(t.dim() != (4 if already_split else 3) for t in tensors):
        return None
    if len({t.shape[0] for t in tensors}) != 1:
        return None
    if already_split:
        return tensors if query.shape[1] == heads else None
    if query.shape[2] % heads:
        return None
    head_dim = query.shape[2] // heads
    if head_dim == 0 or key.shape[2] % head_dim or value.shape[2] % head_dim:
        return None
    kv_heads = key.shape[2] // head_dim
    if value.shape[2] // head_dim != kv_heads:
        return None
    if grouped:
        if kv_heads == 0 or heads % kv_heads:
            return None
    elif kv_heads != heads:
        return None
    return tuple(_split_heads(t, head_dim) for t in tensors)


def _broadcastable_mask(mask):
    """ComfyUI passes (tokens_q, tokens_k) or (batch, tokens_q, tokens_k) masks; attention wants four dimensions."""
    if isinstance(mask, torch.Tensor) and mask.dim() in (2, 3):
        return mask.unsqueeze(0) if mask.dim() == 2 else mask.unsqueeze(1)
    return mask


class ComfyUIAttentionOverride:
    """Callable for `transformer_options["optimized_attention_override"]`.

    `previous_override` is whatever was installed before (called first, with this adapter as its attention function);
    `precision_resolver(attn_precision, dtype)` is ComfyUI's rule for the accumulation precision a call really wants.
    """

    def __init__(self, previous_override=None, precision_resolver=None):
        self.previous_override = previous_override
        self.precision_resolver = precision_resolver if precision_resolver is not None else (lambda wanted, dtype: wanted)

    @staticmethod
    def _fall_back(attention, query, key, value, heads, layout, extra):
        with _bypass_flash_attention():
            return attention(query, key, value, heads, **layout, **extra)

    def _attend(self, comfy_attention, query, key, value, heads, layout, extra):
        grouped = extra.get("enable_gqa") is True
        wants_fp32 = self.precision_resolver(layout["attn_precision"], query.dtype) == torch.float32
        split = _to_head_layout(query, key, value, heads, layout["skip_reshape"], grouped)
        mask = _broadcastable_mask(layout["mask"])
        takes = (split is not None
                 and not (wants_fp32 and query.dtype != torch.float32)
                 and extra.get("low_precision_attention", True) is not False
                 and _is_supported(*split, mask, 0.0, grouped, extra.get("scale")))
        if not takes:
            return self._fall_back(comfy_attention, query, key, value, heads, layout, extra)
        out = flash_attention(*split, softmax_scale=extra.get("scale"), bias=_mask_to_bias(mask))
        if layout["skip_output_reshape"]:
            return out
        batch, _, tokens, head_dim = out.shape
        return out.transpose(1, 2).reshape(batch, tokens, heads * head_dim)

    def __call__(self, comfy_attention, query, key, value, heads, **kwargs):
        layout = {name: kwargs.pop(name, default) for name, default in _LAYOUT_DEFAULTS.items()}
        if self.previous_override is None:
            return self._attend(comfy_attention, query, key, value, heads, layout, kwargs)

        # the earlier override decides; what it is given to delegate to is this adapter around ComfyUI's function
        @wraps(comfy_attention)
        def delegate(q, k, v, n_heads, **inner):
            inner_layout = {name: inner.pop(name, default) for name, default in _LAYOUT_DEFAULTS.items()}
            return self._attend(comfy_attention, q, k, v, n_heads, inner_layout, inner)

        with _bypass_flash_attention():
            return self.previous_override(delegate, query, key, value, heads, **layout, **kwargs)


def _get_comfyui_precision_resolver():
    from comfy.ldm.modules.attention import get_attn_precision

    return get_attn_precision


class ApplyB200FlashAttention:
    """ComfyUI node: returns a clone of the model whose attention calls go through :class:`ComfyUIAttentionOverride`."""

    RETURN_TYPES = ("MODEL",)
    RETURN_NAMES = ("model",)
    FUNCTION = "patch"
    CATEGORY = "model_patches/attention"
    DESCRIPTION = ("Routes this model's supported attention calls through the B200 FlashAttention kernels and falls "
                   "back to ComfyUI's attention for everything else.")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",)}}

    def patch(self, model):
        reason = unsupported_reason()
        if reason is not None:
            raise RuntimeError(f"Cannot enable B200 Flash Attention: {reason}")
        patched = model.clone()
        options = patched.model_options["transformer_options"]
        installed = options.get("optimized_attention_override")
        if installed is not None and not callable(installed):
            raise TypeError("optimized_attention_override must be callable")
        if not isinstance(installed, ComfyUIAttentionOverride):
            if installed is not None:
                logger.info("Composing B200 Flash Attention under an existing attention override")
            options["optimized_attention_override"] = ComfyUIAttentionOverride(installed,
                                                                             _get_comfyui_precision_resolver())
        enable_flash_attention()
        logger.info("Enabled B200 Flash Attention for the patched ComfyUI model")
        return (patched,)


# the reference's node name, for workflows saved against it
ApplyRDNA3FlashAttention = ApplyB200FlashAttention

NODE_CLASS_MAPPINGS = {"ApplyB200FlashAttention": ApplyB200FlashAttention,
                       "ApplyRDNA3FlashAttention": ApplyRDNA3FlashAttention}
NODE_DISPLAY_NAME_MAPPINGS = {"ApplyB200FlashAttention": "B200 Flash Attention",
                              "ApplyRDNA3FlashAttention": "B200 Flash Attention (RDNA3 node name)"}
