"""User-facing attention entry points, signature-compatible with fa_rdna3/interface.py of the reference.

Tensors are ``(batch, heads, seqlen, head_dim)`` as in ``torch.nn.functional.scaled_dot_product_attention``.
Every function allocates its outputs (and scratch) with torch and hands raw pointers, strides and sizes to
the C-ABI library (include/fa_b200.h) on the current CUDA stream; nothing here computes attention itself and
there is no fallback when the library is absent.

Reference entry points mirrored here:
  flash_attention               fa_rdna3/interface.py:355-424
  flash_attention_decode        fa_rdna3/interface.py:427-479
  flash_attention_varlen        fa_rdna3/interface.py:607-640
  flash_attention_decode_paged  fa_rdna3/interface.py:643-728
  alibi_slopes                  fa_rdna3/interface.py:136-151
  ops flash_fwd / flash_bwd / flash_tiny_fwd   fa_rdna3/interface.py:84-104, 283-333
"""
import ctypes as C
import math
import functools
import os
from numbers import Integral

import torch

from . import _lib
from ._validation import (
    LOW_PRECISION_DTYPES,
    SUPPORTED_DTYPES,
    SUPPORTED_HEAD_DIMS,
    validate_attention_options,
    validate_dense_inputs,
    validate_inference_only,
    validate_paged_inputs,
    validate_softmax_scale,
    validate_varlen_inputs,
)

_SUPPORTED_HEAD_DIMS = SUPPORTED_HEAD_DIMS
_SUPPORTED_DTYPES = SUPPORTED_DTYPES

# Split-K decode aims at four CTAs per SM; a B200 has 148 SMs. Used only as the default of
# _decode_num_splits; the public call passes 4 x the device's real SM count.
_DECODE_TARGET_PROGRAMS = 4 * 148
_DECODE_BLOCK_M = 16

_DTYPE_CODE = {torch.float16: _lib.FA_F16, torch.bfloat16: _lib.FA_BF16, torch.float32: _lib.FA_F32}


def _cdiv(a, b):
    return -(-a // b)


def _next_power_of_2(n):
    return 1 if n <= 1 else 1 << (int(n) - 1).bit_length()


def _decode_num_splits(batch, heads, seqlen_q, seqlen_k, target_programs=_DECODE_TARGET_PROGRAMS):
    """Number of key slices for split-K decode (fa_rdna3/interface.py:53-58): enough programs to fill
    the GPU, at most 32, and never slices shorter than 64 keys."""
    base = batch * heads * _cdiv(seqlen_q, _DECODE_BLOCK_M)
    wanted = _cdiv(target_programs, base)
    return max(1, min(32, wanted, _cdiv(seqlen_k, 64)))


def _paged_num_splits(batch, heads, block_size, max_blocks, target_programs,
                      max_context_len=None, requested_splits=None):
    """Split count of paged decode (fa_rdna3/interface.py:61-77)."""
    if requested_splits is not None:
        return requested_splits
    if max_context_len is None:
        active_blocks = max_blocks
        active_tokens = max_blocks * block_size
    else:
        active_blocks = min(max_blocks, _cdiv(max_context_len, block_size))
        active_tokens = min(max_blocks * block_size, max_context_len)
    if active_tokens <= 64:
        return 1
    cap = min(16, active_blocks, target_programs)
    by_occupancy = _cdiv(5 * target_programs, batch * heads)
    by_work = min(16, _cdiv(active_tokens, 256))
    return min(cap, max(by_occupancy, by_work))


@functools.lru_cache(maxsize=4096)
def _fill_splits(base_ctas, max_splits, sm_count, ctas_per_sm=2):
    """Split count for the B200 decode kernels: the grid is `base_ctas * splits` CTAs and `ctas_per_sm * sm_count`
    of them are resident at once, so pick the split count whose last wave is fullest (fewest splits within 3 %
    of the best fill), once there is at least one full wave."""
    slots = ctas_per_sm * sm_count
    max_splits = max(1, int(max_splits))
    best, best_fill = 1, -1.0
    for s in range(1, max_splits + 1):
        ctas = base_ctas * s
        fill = ctas / (_cdiv(ctas, slots) * slots)
        if ctas < slots and s < max_splits:
            continue                      # not even one wave yet: keep splitting
        if fill > best_fill + 0.03:
            best, best_fill = s, fill
    return best


def _decode_splits_b200(batch, kv_heads, group_rows, seqlen_k, sm_count, tensor_core=False, head_dim=128):
    """Key slices for split-K decode on B200. Tensor-core kernel: one CTA per SM, every CTA walks two streams of
    128-key tiles and emits two partials, so the count is even and each CTA gets at least two tiles.
    CUDA-core kernel: CTAs are per (batch, kv head, chunk of 4 query rows), two per SM; slices are at least 512
    keys long and at most 64."""
    if tensor_core:
        tiles = _cdiv(seqlen_k, 128)
        # one wave of long CTAs beats several waves of short ones (per-CTA start-up is not amortised otherwise)
        heads = batch * kv_heads
        ctas = max(1, sm_count // heads) if heads < sm_count else 1
        if head_dim > 128:  # one stream and one partial per CTA; the kernel wants at least two partials
            return max(2, min(ctas, 32, max(1, tiles // 2)))
        return 2 * min(ctas, 32, max(1, tiles // 2))
    rows_per_cta = 1 if group_rows == 1 else 2 if group_rows == 2 else 4
    base = batch * kv_heads * _cdiv(group_rows, rows_per_cta)
    return _fill_splits(base, min(64, max(1, seqlen_k // 512)), sm_count)


def _paged_splits_b200(batch, kv_heads, group, block_size, max_blocks, sm_count, max_context_len=None,
                       tensor_core=False):
    """Splits of paged decode on B200 (at most 32, each at least 256 tokens of the longest context); the
    tensor-core kernel takes an even count, two partials per CTA, one CTA per SM."""
    tokens = max_blocks * block_size if max_context_len is None else min(max_blocks * block_size, max_context_len)
    if tensor_core:
        # one CTA row per batch entry; a 128-row tile holds 128 / kv_heads tokens of all kv heads
        tiles = _cdiv(tokens * kv_heads, 128)
        return 2 * _fill_splits(batch, min(64, max(1, tiles // 2)), sm_count, ctas_per_sm=1)
    rows_per_cta = 1 if group == 1 else 2 if group == 2 else 4
    base = batch * kv_heads * _cdiv(group, rows_per_cta)
    return _fill_splits(base, min(32, max(1, tokens // 256)), sm_count)


def _paged_balanced_slots(kv_heads, block_size, max_blocks, sm_count, max_context_len=None):
    """Partial slots per sequence for the balanced tensor-core paged kernel: two per CTA, and a sequence never gets
    more CTAs than half its 128-row tiles (a tile holds 128 / kv_heads tokens of all kv heads) or than there are SMs."""
    tokens = max_blocks * block_size if max_context_len is None else min(max_blocks * block_size, max_context_len)
    tiles = _cdiv(tokens * kv_heads, 128)
    return 2 * max(1, min(sm_count, tiles // 2))


def alibi_slopes(n_heads, device="cuda"):
    """Standard ALiBi per-head slopes (Press et al., 2021) as an fp32 ``(n_heads,)`` tensor
    (fa_rdna3/interface.py:136-151)."""
    if isinstance(n_heads, bool) or not isinstance(n_heads, Integral) or n_heads <= 0:
        raise ValueError("n_heads must be a positive integer")

    def geometric(n):
        ratio = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [ratio ** (i + 1) for i in range(n)]

    if n_heads & (n_heads - 1) == 0:
        slopes = geometric(n_heads)
    else:
        lower = 1 << (n_heads.bit_length() - 1)
        slopes = geometric(lower) + geometric(2 * lower)[0::2][: n_heads - lower]
    return torch.tensor(slopes, dtype=torch.float32, device=device)


def _bias_args(bias, query, batch, heads, seqlen_q, seqlen_k):
    """(tensor, sbb, sbh, sbm, sbn, has_bias) for a kernel call (fa_rdna3/interface.py:115-126): a present
    bias is expanded, never materialised, so broadcast dimensions carry stride 0."""
    if bias is None:
        return query, 0, 0, 0, 0, False
    bias = bias.expand(batch, heads, seqlen_q, seqlen_k)
    sbb, sbh, sbm, sbn = bias.stride()
    return bias, sbb, sbh, sbm, sbn, True


def _alibi_args(alibi_slopes, query):
    if alibi_slopes is None:
        return query, False
    return alibi_slopes.to(torch.float32).contiguous(), True


# ---------------------------------------------------------------------------------------------------
# plumbing to the C ABI
# ---------------------------------------------------------------------------------------------------
_status_words = {}


def _status_word(device):
    """One int32 per device that kernels set when a bounded internal wait ran out."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status_words[key] = word
    return word


def check_status(device=None):
    """Synchronise and raise if any kernel on `device` reported a lost wait since the last check."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    word = _status_words.get(index)
    if word is None:
        return
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"fa_b200 kernel reported an internal wait timeout (code {code})")


def _stream(device):
    """The raw handle of torch's current stream on `device` (the private accessor is several times cheaper than
    building a Stream object per launch; the public route is the fall-back)."""
    index = device.index if isinstance(device, torch.device) else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    try:
        return C.c_void_p(torch._C._cuda_getCurrentRawStream(index))
    except AttributeError:
        return C.c_void_p(torch.cuda.current_stream(index).cuda_stream)


def _set4(field, strides):
    for i, s in enumerate(strides):
        field[i] = int(s)


def _strides_bhsd(t, varlen):
    """Element strides ordered (batch, head, seq, dim); packed tensors are (token, head, dim)."""
    if varlen:
        st, sh, sd = t.stride()
        return (0, sh, st, sd)
    return t.stride()


def _attn_params(query, key, value, out, lse, causal, softmax_scale, window, softcap, bias, alibi,
                 dropout_p, dropout_seed, *, varlen=None, force_path=0):
    p = _lib.AttnParams()
    p.dtype = _DTYPE_CODE[query.dtype]
    is_varlen = varlen is not None
    p.varlen = int(is_varlen)
    if is_varlen:
        cu_q, cu_k, max_q, max_k = varlen
        p.batch = cu_q.numel() - 1
        p.heads_q, p.heads_kv = query.shape[1], key.shape[1]
        p.seqlen_q, p.seqlen_k = int(max_q), int(max_k)
        p.total_q, p.total_k = query.shape[0], key.shape[0]
        p.head_dim = query.shape[2]
        p.cu_seqlens_q = cu_q.data_ptr()
        p.cu_seqlens_k = cu_k.data_ptr()
        lse_strides = (0, lse.stride(0), lse.stride(1))
    else:
        p.batch, p.heads_q, p.seqlen_q, p.head_dim = query.shape
        p.heads_kv, p.seqlen_k = key.shape[1], key.shape[2]
        lse_strides = lse.stride()
    p.q, p.k, p.v, p.out, p.lse = query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), lse.data_ptr()
    _set4(p.q_strides, _strides_bhsd(query, is_varlen))
    _set4(p.k_strides, _strides_bhsd(key, is_varlen))
    _set4(p.v_strides, _strides_bhsd(value, is_varlen))
    _set4(p.o_strides, _strides_bhsd(out, is_varlen))
    _set4(p.lse_strides, lse_strides)
    p.softmax_scale = float(softmax_scale)
    p.softcap = float(softcap)
    if bias is not None:
        bias_t, sbb, sbh, sbm, sbn, _ = _bias_args(bias, query, p.batch, p.heads_q, p.seqlen_q, p.seqlen_k)
        p.bias = bias_t.data_ptr()
        p.bias_dtype = _DTYPE_CODE[bias_t.dtype]
        _set4(p.bias_strides, (sbb, sbh, sbm, sbn))
    if alibi is not None:
        p.alibi_slopes = alibi.data_ptr()
    p.causal = int(bool(causal))
    p.window_left, p.window_right = int(window[0]), int(window[1])
    p.dropout_p = float(dropout_p)
    p.dropout_seed = int(dropout_seed)
    p.status = _status_word(query.device).data_ptr()
    p.force_path = int(force_path)
    return p


_force_path = 0


class force_kernel_path:
    """Context manager for tests: force the tensor-core ("tcgen05") or CUDA-core ("simt") kernels."""

    def __init__(self, name):
        self.value = {"auto": 0, "tcgen05": _lib.FA_PATH_TCGEN05, "simt": _lib.FA_PATH_SIMT}[name]

    def __enter__(self):
        global _force_path
        self.previous = _force_path
        _force_path = self.value

    def __exit__(self, *exc):
        global _force_path
        _force_path = self.previous


def last_kernel_path():
    """"tcgen05", "simt" or "none": the kernel family of this thread's last forward/backward call."""
    return {0: "none", 1: "tcgen05", 2: "simt"}[_lib.load().fa_last_path()]


def _forward(query, key, value, causal, softmax_scale, window, softcap, bias, alibi, dropout_p, dropout_seed):
    """Dense forward launch: allocates O and LSE, returns (out, lse) (fa_rdna3/interface.py:154-199)."""
    lib = _lib.load()
    batch, heads, seqlen_q, head_dim = query.shape
    out = torch.empty_like(query)
    lse = torch.empty((batch, heads, seqlen_q), dtype=torch.float32, device=query.device)
    alibi_t = None if alibi is None else _alibi_args(alibi, query)[0]
    # head dims above 256 run on the tensor cores when they get a scratch for their P tiles (2 bytes per score; no score
    # modifier): a batch whose scratch exceeds the limit goes entry by entry
    plain = softcap == 0.0 and bias is None and alibi is None and dropout_p == 0.0
    fp32_tc = plain and FP32_ON_TENSOR_CORES and query.dtype == torch.float32 and head_dim <= 256 and head_dim % 8 == 0
    pieces = _wide_batch_pieces(query, key, 1, 256) if plain else [(0, batch)]
    for b0, b1 in pieces:
        sl = slice(b0, b1)
        bias_piece = bias[sl] if (bias is not None and bias.dim() == 4 and bias.shape[0] > 1) else bias
        p = _attn_params(query[sl], key[sl], value[sl], out[sl], lse[sl], causal, softmax_scale, window, softcap,
                         bias_piece, alibi_t, dropout_p, dropout_seed, force_path=_force_path)
        ws = _scratch(p, _lib.FA_WS_FWD_P, query.device) if (plain and (head_dim > 256 or fp32_tc)) else None  # noqa: F841
        with torch.cuda.device(query.device):
            _lib.check(lib.fa_fwd(C.byref(p), _stream(query.device)))
    return out, lse


def _fill_backward(p, dout, delta, dq, dk, dv, is_varlen):
    p.dout, p.delta, p.dq, p.dk, p.dv = dout.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    _set4(p.do_strides, _strides_bhsd(dout, is_varlen))
    _set4(p.dq_strides, _strides_bhsd(dq, is_varlen))
    _set4(p.dk_strides, _strides_bhsd(dk, is_varlen))
    _set4(p.dv_strides, _strides_bhsd(dv, is_varlen))
    _set4(p.delta_strides, (0, delta.stride(0), delta.stride(1)) if is_varlen else delta.stride())


# The dense backward may keep dS (16 bits per score of every query head) in a scratch buffer so that dQ becomes one
# GEMM instead of a second pass that recomputes the scores; above this many bytes it does not (set to 0 to switch the
# scratch form off; the result is the same either way).
DS_WORKSPACE_LIMIT_BYTES = int(os.environ.get("FA_B200_DS_WORKSPACE_MB", "512")) << 20
# Head dims above 128 have no tensor-core backward without the scratch (it then holds P and dS, 4 bytes per score), and
# the CUDA-core kernels are 50 times slower: the limit is higher, and a batch that does not fit is taken in pieces.
DS_WORKSPACE_WIDE_LIMIT_BYTES = int(os.environ.get("FA_B200_DS_WORKSPACE_WIDE_MB", "4096")) << 20


# fp32 inputs run exact fp32 arithmetic on the CUDA cores (2e-5 against fp64 math) unless this is switched on: then
# the dense forward without score modifiers, head dims to 256, computes Q K^T as tf32 products and P V in fp16 on the
# tensor cores (about 1e-3 absolute error on N(0,1) inputs, inside the 2e-3 / 3e-3 the reference's own fp32 tests allow,
# fa_rdna3 tests/test_fp32_headdim.py:35-53; V must stay inside the fp16 range). Off by default: a caller who passes
# fp32 asked for fp32. The backward of fp32 inputs is exact either way.
FP32_ON_TENSOR_CORES = os.environ.get("FA_B200_FP32_TENSOR_CORES", "0") == "1"

_poison_ds_workspace = False


def _scratch(p, kind, device):
    """Scratch of `kind` for the problem in `p`, or None when the problem does not take one or it would be larger than
    the limit for its head dim. Attached to `p`; the caller keeps the returned tensor alive."""
    need = _lib.load().fa_workspace_bytes(kind, C.byref(p))
    limit = (DS_WORKSPACE_WIDE_LIMIT_BYTES if (p.head_dim > 128 or kind == _lib.FA_WS_FWD_P or p.dtype == _lib.FA_F32)
             else DS_WORKSPACE_LIMIT_BYTES)
    if need <= 0 or need > limit:
        return None
    ws = torch.empty(need + 1024, dtype=torch.uint8, device=device)
    if _poison_ds_workspace:
        ws.fill_(0xFF)   # tests: every 16-bit word a NaN, so a tile that is read without having been written shows
    base = (ws.data_ptr() + 1023) & ~1023
    p.ds_workspace, p.ds_workspace_bytes = base, need
    return ws


def _ds_workspace(p, device):
    """Scratch for the dS form of the dense backward (see _scratch). fp32 inputs only get one (and with it tensor-core
    products) when FP32_ON_TENSOR_CORES is on."""
    if p.dtype == _lib.FA_F32 and not FP32_ON_TENSOR_CORES:
        return None
    return _scratch(p, _lib.FA_WS_BWD_DS, device)


def _wide_batch_pieces(query, key, tiles_per_pair, above):
    """Batch ranges of one launch each. One range, except for 16-bit head dims above `above` whose scratch
    (`tiles_per_pair` 32 KB tiles per 128 x 128 block of scores of every query head) exceeds its limit: those go batch
    entry by batch entry, as many per launch as fit."""
    batch, heads, seqlen_q, head_dim = query.shape
    whole = [(0, batch)]
    if head_dim <= above or head_dim > 512 or query.dtype not in (torch.float16, torch.bfloat16):
        return whole
    qt = -(-seqlen_q // 128)
    per_entry = heads * (tiles_per_pair * qt * (-(-key.shape[2] // 128)) * 32768 + (qt * 1024 if above == 256 else 0))
    if per_entry * batch <= DS_WORKSPACE_WIDE_LIMIT_BYTES or per_entry > DS_WORKSPACE_WIDE_LIMIT_BYTES:
        return whole
    step = DS_WORKSPACE_WIDE_LIMIT_BYTES // per_entry
    return [(b0, min(b0 + step, batch)) for b0 in range(0, batch, step)]


def _backward(dout, query, key, value, out, lse, causal, softmax_scale, window, softcap, bias, alibi,
              dropout_p, dropout_seed):
    """Dense backward launch: returns (dq, dk, dv) (fa_rdna3/interface.py:202-277)."""
    lib = _lib.load()
    dout = dout.contiguous()
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)
    alibi_t = None if alibi is None else _alibi_args(alibi, query)[0]
    # dropout counters depend on the batch index inside a launch, so a problem with dropout is never cut
    for b0, b1 in (_wide_batch_pieces(query, key, 2, 128) if dropout_p == 0.0 else [(0, query.shape[0])]):
        sl = slice(b0, b1)
        bias_piece = bias[sl] if (bias is not None and bias.dim() == 4 and bias.shape[0] > 1) else bias
        p = _attn_params(query[sl], key[sl], value[sl], out[sl], lse[sl], causal, softmax_scale, window, softcap,
                         bias_piece, alibi_t, dropout_p, dropout_seed, force_path=_force_path)
        _fill_backward(p, dout[sl], delta[sl], dq[sl], dk[sl], dv[sl], False)
        ws = _ds_workspace(p, query.device)  # noqa: F841  (kept alive until the launch below is queued)
        with torch.cuda.device(query.device):
            _lib.check(lib.fa_bwd(C.byref(p), _stream(query.device)))
    return dq, dk, dv


# Registered as torch.library custom ops so they are opaque to torch.compile, carry fake kernels and an
# autograd rule, and stay functional: the dropout seed is an input, not hidden state
# (fa_rdna3/interface.py:280-333).
@torch.library.custom_op("fa_b200::flash_fwd", mutates_args=())
def _flash_fwd(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
               causal: bool, softmax_scale: float, window_left: int, window_right: int,
               softcap: float, bias: "torch.Tensor | None", alibi: "torch.Tensor | None",
               dropout_p: float, dropout_seed: int) -> "tuple[torch.Tensor, torch.Tensor]":
    return _forward(query, key, value, causal, softmax_scale, (window_left, window_right),
                    softcap, bias, alibi, dropout_p, dropout_seed)


@_flash_fwd.register_fake
def _(query, key, value, causal, softmax_scale, window_left, window_right,
      softcap, bias, alibi, dropout_p, dropout_seed):
    out = torch.empty_like(query)
    lse = query.new_empty((query.shape[0], query.shape[1], query.shape[2]), dtype=torch.float32)
    return out, lse


@torch.library.custom_op("fa_b200::flash_bwd", mutates_args=())
def _flash_bwd(dout: torch.Tensor, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
               out: torch.Tensor, lse: torch.Tensor, causal: bool, softmax_scale: float,
               window_left: int, window_right: int, softcap: float,
               bias: "torch.Tensor | None", alibi: "torch.Tensor | None",
               dropout_p: float, dropout_seed: int) -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    return _backward(dout, query, key, value, out, lse, causal, softmax_scale,
                     (window_left, window_right), softcap, bias, alibi, dropout_p, dropout_seed)


@_flash_bwd.register_fake
def _(dout, query, key, value, out, lse, causal, softmax_scale, window_left, window_right,
      softcap, bias, alibi, dropout_p, dropout_seed):
    return torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)


def _flash_fwd_setup_context(ctx, inputs, output):
    (query, key, value, causal, softmax_scale, window_left, window_right,
     softcap, bias, alibi, dropout_p, dropout_seed) = inputs
    out, lse = output
    ctx.save_for_backward(query, key, value, out, lse, bias, alibi)
    ctx.args = (causal, softmax_scale, window_left, window_right, softcap, dropout_p, dropout_seed)


def _flash_fwd_backward(ctx, grad_out, grad_lse):
    query, key, value, out, lse, bias, alibi = ctx.saved_tensors
    causal, softmax_scale, window_left, window_right, softcap, dropout_p, dropout_seed = ctx.args
    dq, dk, dv = _flash_bwd(grad_out.contiguous(), query, key, value, out, lse, causal, softmax_scale,
                            window_left, window_right, softcap, bias, alibi, dropout_p, dropout_seed)
    return dq, dk, dv, None, None, None, None, None, None, None, None, None


_flash_fwd.register_autograd(_flash_fwd_backward, setup_context=_flash_fwd_setup_context)


@torch.library.custom_op("fa_b200::flash_tiny_fwd", mutates_args=())
def _flash_tiny_fwd(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    softmax_scale: float, bias: "torch.Tensor | None", block_n: int) -> torch.Tensor:
    """FP32 short-sequence forward (fa_rdna3/interface.py:84-104). ``block_n`` is kept for schema
    compatibility; the CUDA kernel always keeps one score per lane."""
    lib = _lib.load()
    batch, heads, seqlen, head_dim = query.shape
    out = torch.empty_like(query)
    p = _lib.TinyParams()
    p.batch, p.heads, p.seqlen, p.head_dim = batch, heads, seqlen, head_dim
    p.q, p.k, p.v, p.out = query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr()
    _set4(p.q_strides, query.stride())
    _set4(p.k_strides, key.stride())
    _set4(p.v_strides, value.stride())
    _set4(p.o_strides, out.stride())
    bias_t, sbb, sbh, sbm, sbn, has_bias = _bias_args(bias, query, batch, heads, seqlen, seqlen)
    if has_bias:
        p.bias = bias_t.data_ptr()
        p.bias_dtype = _DTYPE_CODE[bias_t.dtype]
        _set4(p.bias_strides, (sbb, sbh, sbm, sbn))
    p.softmax_scale = float(softmax_scale)
    with torch.cuda.device(query.device):
        _lib.check(lib.fa_tiny_fwd(C.byref(p), _stream(query.device)))
    return out


@_flash_tiny_fwd.register_fake
def _(query, key, value, softmax_scale, bias, block_n):
    return torch.empty_like(query)


def _can_use_tiny_forward(query, key, value, causal, window_size, softcap,
                          alibi_slopes, dropout_p, head_dim):
    """Routing predicate of the FP32 short-sequence kernel (fa_rdna3/interface.py:336-352)."""
    requires_backward = torch.is_grad_enabled() and (
        query.requires_grad or key.requires_grad or value.requires_grad)
    return (
        not requires_backward
        and query.dtype == torch.float32
        and head_dim == 128
        and query.shape[1] == key.shape[1] == value.shape[1]
        and query.shape[2] == key.shape[2] == value.shape[2]
        and query.shape[2] <= 32
        and not causal
        and window_size == (-1, -1)
        and softcap == 0.0
        and alibi_slopes is None
        and dropout_p == 0.0
    )


def flash_attention(query, key, value, causal=False, softmax_scale=None, window_size=(-1, -1),
                    softcap=0.0, bias=None, alibi_slopes=None, dropout_p=0.0):
    """Scaled dot-product attention on B200 tensor cores; differentiable in q, k, v.

    Args:
        query, key, value: ``(batch, heads, seqlen, head_dim)`` in float16, bfloat16 or float32; key and
            value may have fewer heads (grouped-query attention).
        causal: causal mask, bottom-right aligned when the sequence lengths differ.
        softmax_scale: logit scale, default ``1/sqrt(head_dim)``.
        window_size: ``(left, right)``; query ``i`` sees keys ``i - left <= j <= i + right``; ``-1`` = no limit.
        softcap: if > 0, logits become ``softcap * tanh(logit / softcap)``.
        bias: additive logit bias broadcastable to ``(batch, heads, seqlen_q, seqlen_k)`` (``-inf`` masks);
            not differentiable.
        alibi_slopes: ``(heads,)`` ALiBi slopes, adds ``-slope * |query_pos - key_pos|``.
        dropout_p: attention dropout probability; the seed is drawn per forward and reused in backward.

    Same contract as fa_rdna3/interface.py:355-424 of the reference.
    """
    validate_dense_inputs(query, key, value)
    validate_attention_options(
        query, key, softmax_scale=softmax_scale, window_size=window_size, softcap=softcap,
        bias=bias, alibi_slopes=alibi_slopes, dropout_p=dropout_p)
    head_dim = query.shape[-1]
    softmax_scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    window_size = tuple(window_size)
    softcap = float(softcap)
    dropout_p = float(dropout_p)

    if _can_use_tiny_forward(query, key, value, causal, window_size, softcap, alibi_slopes, dropout_p, head_dim):
        seqlen = query.shape[2]
        block_n = 8 if seqlen <= 8 else 16 if seqlen <= 16 else 32
        return _flash_tiny_fwd(query, key, value, softmax_scale, bias, block_n)

    # Head dims that are not a supported power of two are zero-padded (zeros add nothing to q.k or p.v)
    # and the output is sliced back; pad and slice are autograd-tracked.
    # 16-bit head dims that are a multiple of 8 up to 256 need no copy: the tensor-core kernels read the narrower rows
    # through their tensor maps, which fill the columns up to 64, 128 or 256 with zeros (above 128 the backward runs
    # on the CUDA-core kernels, which take any width).
    pad = 0
    padded = head_dim
    direct = query.dtype in LOW_PRECISION_DTYPES and head_dim % 8 == 0 and head_dim <= 256
    if not direct and head_dim not in _SUPPORTED_HEAD_DIMS:
        padded = max(16, _next_power_of_2(head_dim))
        if padded not in _SUPPORTED_HEAD_DIMS:
            raise ValueError(f"head_dim {head_dim} not supported (would pad to {padded})")
    if padded != head_dim:
        pad = padded - head_dim
        query = torch.nn.functional.pad(query, (0, pad))
        key = torch.nn.functional.pad(key, (0, pad))
        value = torch.nn.functional.pad(value, (0, pad))

    dropout_seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item()) if dropout_p > 0.0 else 0
    out, _ = _flash_fwd(query, key, value, causal, softmax_scale, window_size[0], window_size[1],
                        softcap, bias, alibi_slopes, dropout_p, dropout_seed)
    return out[..., :head_dim] if pad else out


def _vector_friendly(t):
    """True when rows of `t` can be read with 16-byte loads (unit inner stride, aligned rows)."""
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    return all(s % 8 == 0 for s, n in zip(t.stride()[:-1], t.shape[:-1]) if n > 1)


_copy_warned = set()


def _rows_readable(t, what):
    """The decode kernels read K/V rows with 16-byte loads. A cache whose layout does not allow that (inner stride
    not 1, or rows not 16-byte aligned) is accepted, as the reference accepts any strides, but it costs a copy of the
    whole cache on every call: say so once per call site instead of hiding it."""
    if _vector_friendly(t):
        return t
    if what not in _copy_warned:
        _copy_warned.add(what)
        import warnings

        warnings.warn(f"fa_b200: {what} is not readable with 16-byte loads (strides {tuple(t.stride())}); it is copied "
                      "to a contiguous tensor on every call. Pass caches with unit inner stride and rows aligned to "
                      "16 bytes to avoid the copy.", RuntimeWarning, stacklevel=3)
    return t.contiguous()


def _tensor_core_decode_ok(query, head_dim, rows_per_kv_head, softmax_scale):
    """Host-side mirror of the tcgen05 decode kernel's shape limits (the library re-checks strides itself)."""
    if head_dim == 256 and rows_per_kv_head < 4:  # the library keeps these on the CUDA-core kernel (faster there)
        return False
    return (query.dtype in LOW_PRECISION_DTYPES and head_dim in (64, 128, 256) and rows_per_kv_head <= 128
            and softmax_scale > 0)


def _paged_tensor_core_ok(query, head_dim, q_heads, kv_heads, block_size, softmax_scale):
    """Shape limits of the tcgen05 paged kernel: every query head is one MMA row, kv heads interleave in a tile."""
    return (query.dtype in LOW_PRECISION_DTYPES and head_dim in (64, 128) and q_heads <= 128 and softmax_scale > 0
            and kv_heads & (kv_heads - 1) == 0 and block_size * kv_heads >= 8)


def _decode_impl(query, key, value, softmax_scale, num_splits, force_path=0):
    lib = _lib.load()
    batch, heads, seqlen_q, head_dim = query.shape
    key = _rows_readable(key, "the key cache of flash_attention_decode")
    value = _rows_readable(value, "the value cache of flash_attention_decode")
    out = torch.empty_like(query)
    p = _lib.DecodeParams()
    p.dtype = _DTYPE_CODE[query.dtype]
    p.batch, p.heads_q, p.heads_kv = batch, heads, key.shape[1]
    p.seqlen_q, p.seqlen_k, p.head_dim = seqlen_q, key.shape[2], head_dim
    p.q, p.k, p.v, p.out = query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr()
    _set4(p.q_strides, query.stride())
    _set4(p.k_strides, key.stride())
    _set4(p.v_strides, value.stride())
    _set4(p.o_strides, out.stride())
    p.softmax_scale = float(softmax_scale)
    p.num_splits = int(num_splits)
    p.force_path = int(force_path)
    p.status = _status_word(query.device).data_ptr()
    if num_splits > 1:
        o_partial = torch.empty((num_splits, batch, heads, seqlen_q, head_dim), dtype=torch.float32,
                                device=query.device)
        lse_partial = torch.empty((num_splits, batch, heads, seqlen_q), dtype=torch.float32, device=query.device)
        p.o_partial, p.lse_partial = o_partial.data_ptr(), lse_partial.data_ptr()
    with torch.cuda.device(query.device):
        _lib.check(lib.fa_decode_splitk(C.byref(p), _stream(query.device)))
    return out


@torch.library.custom_op("fa_b200::decode_splitk", mutates_args=())
def _decode_op(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, softmax_scale: float,
               num_splits: int) -> torch.Tensor:
    return _decode_impl(query, key, value, softmax_scale, num_splits)


@_decode_op.register_fake
def _(query, key, value, softmax_scale, num_splits):
    return torch.empty_like(query)


def flash_attention_decode(query, key, value, softmax_scale=None):
    """Split-K attention for autoregressive decode: a short query against a long KV cache, the cache cut
    into slices that run on different SMs and are merged with an LSE reduction. Non-causal, inference-only.
    Same contract as fa_rdna3/interface.py:427-479."""
    validate_dense_inputs(query, key, value, dtypes=LOW_PRECISION_DTYPES)
    validate_inference_only(query, key, value)
    validate_softmax_scale(softmax_scale)
    batch, heads, seqlen_q, head_dim = query.shape
    seqlen_k = key.shape[2]
    if head_dim not in _SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head_dim {head_dim} not supported; expected one of {_SUPPORTED_HEAD_DIMS}")
    softmax_scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    # The reference sizes its grid per query head (_decode_num_splits above); these kernels run one CTA per kv head
    # and slice of keys, so the count comes from the B200 grid-fill rule instead.
    sm_count = torch.cuda.get_device_properties(query.device).multi_processor_count
    rows = (heads // key.shape[1]) * seqlen_q
    num_splits = _decode_splits_b200(batch, key.shape[1], rows, seqlen_k, sm_count,
                                     tensor_core=_tensor_core_decode_ok(query, head_dim, rows, softmax_scale),
                                     head_dim=head_dim)
    return _decode_op(query, key, value, softmax_scale, num_splits)


# ---------------------------------------------------------------------------------------------------
# packed variable-length attention
# ---------------------------------------------------------------------------------------------------
def _forward_varlen(query, key, value, cu_seqlens_q, cu_seqlens_k,
                    max_seqlen_q, max_seqlen_k, causal, softmax_scale, window, softcap, alibi):
    """Packed forward launch: returns (out, lse) with lse shaped (q_heads, total_q)
    (fa_rdna3/interface.py:482-511)."""
    lib = _lib.load()
    total_q, q_heads, _ = query.shape
    out = torch.empty_like(query)
    lse = torch.empty((q_heads, total_q), dtype=torch.float32, device=query.device)
    alibi_t = None if alibi is None else _alibi_args(alibi, query)[0]
    p = _attn_params(query, key, value, out, lse, causal, softmax_scale, window, softcap, None, alibi_t, 0.0, 0,
                     varlen=(cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k), force_path=_force_path)
    with torch.cuda.device(query.device):
        _lib.check(lib.fa_varlen_fwd(C.byref(p), _stream(query.device)))
    return out, lse


def _backward_varlen(dout, query, key, value, out, lse, cu_seqlens_q, cu_seqlens_k,
                     max_seqlen_q, max_seqlen_k, causal, softmax_scale, window, softcap, alibi):
    """Packed backward launch (fa_rdna3/interface.py:514-580). Rows outside every sequence get zero
    gradients."""
    lib = _lib.load()
    dout = dout.contiguous()
    # zeros, not empty: the packed tensors may hold rows that belong to no sequence (cu_seqlens need not cover them,
    # and out-of-range entries are clamped), which no kernel visits and whose gradients are zero by definition
    delta = torch.zeros_like(lse)
    dq, dk, dv = torch.zeros_like(query), torch.zeros_like(key), torch.zeros_like(value)
    alibi_t = None if alibi is None else _alibi_args(alibi, query)[0]
    p = _attn_params(query, key, value, out, lse, causal, softmax_scale, window, softcap, None, alibi_t, 0.0, 0,
                     varlen=(cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k), force_path=_force_path)
    _fill_backward(p, dout, delta, dq, dk, dv, True)
    with torch.cuda.device(query.device):
        _lib.check(lib.fa_varlen_bwd(C.byref(p), _stream(query.device)))
    return dq, dk, dv


@torch.library.custom_op("fa_b200::varlen_fwd", mutates_args=())
def _varlen_fwd(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                causal: bool, softmax_scale: float, window_left: int, window_right: int, softcap: float,
                alibi: "torch.Tensor | None") -> "tuple[torch.Tensor, torch.Tensor]":
    return _forward_varlen(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                           causal, softmax_scale, (window_left, window_right), softcap, alibi)


@_varlen_fwd.register_fake
def _(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, softmax_scale,
      window_left, window_right, softcap, alibi):
    return torch.empty_like(query), query.new_empty((query.shape[1], query.shape[0]), dtype=torch.float32)


@torch.library.custom_op("fa_b200::varlen_bwd", mutates_args=())
def _varlen_bwd(dout: torch.Tensor, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                out: torch.Tensor, lse: torch.Tensor, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                max_seqlen_q: int, max_seqlen_k: int, causal: bool, softmax_scale: float,
                window_left: int, window_right: int, softcap: float,
                alibi: "torch.Tensor | None") -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    return _backward_varlen(dout, query, key, value, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                            max_seqlen_k, causal, softmax_scale, (window_left, window_right), softcap, alibi)


@_varlen_bwd.register_fake
def _(dout, query, key, value, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal,
      softmax_scale, window_left, window_right, softcap, alibi):
    return torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)


def _varlen_setup_context(ctx, inputs, output):
    (query, key, value, cu_q, cu_k, max_q, max_k, causal, softmax_scale, wl, wr, softcap, alibi) = inputs
    out, lse = output
    ctx.save_for_backward(query, key, value, out, lse, cu_q, cu_k, alibi)
    ctx.args = (max_q, max_k, causal, softmax_scale, wl, wr, softcap)


def _varlen_backward(ctx, grad_out, grad_lse):
    query, key, value, out, lse, cu_q, cu_k, alibi = ctx.saved_tensors
    max_q, max_k, causal, softmax_scale, wl, wr, softcap = ctx.args
    dq, dk, dv = _varlen_bwd(grad_out.contiguous(), query, key, value, out, lse, cu_q, cu_k, max_q, max_k,
                             causal, softmax_scale, wl, wr, softcap, alibi)
    return dq, dk, dv, None, None, None, None, None, None, None, None, None, None


_varlen_fwd.register_autograd(_varlen_backward, setup_context=_varlen_setup_context)


def flash_attention_varlen(query, key, value, cu_seqlens_q, cu_seqlens_k,
                           max_seqlen_q, max_seqlen_k, causal=False, softmax_scale=None,
                           window_size=(-1, -1), softcap=0.0, alibi_slopes=None):
    """Attention over variable-length sequences packed without padding; differentiable in q, k, v.

    query is ``(total_q, q_heads, head_dim)``, key/value ``(total_k, kv_heads, head_dim)``;
    ``cu_seqlens_*`` are int32 ``(batch + 1,)`` cumulative lengths. Masks and modifiers apply per
    sequence. Same contract as fa_rdna3/interface.py:607-640.
    """
    validate_varlen_inputs(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k)
    validate_attention_options(
        query, key, softmax_scale=softmax_scale, window_size=window_size, softcap=softcap,
        bias=None, alibi_slopes=alibi_slopes, dropout_p=0.0)
    head_dim = query.shape[-1]
    softmax_scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    window_size = tuple(window_size)
    out, _ = _varlen_fwd(query, key, value, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k),
                         bool(causal), softmax_scale, int(window_size[0]), int(window_size[1]), float(softcap),
                         alibi_slopes)
    return out


# ---------------------------------------------------------------------------------------------------
# paged-KV decode
# ---------------------------------------------------------------------------------------------------
def _paged_launch(query, k_cache, v_cache, block_table, context_lens, softmax_scale, num_splits,
                  first_block=0, block_step=1, want_lse=False, out_f32=False, force_path=0, balance=False,
                  out_buffers=None):
    """Launch paged decode over logical blocks first_block, first_block + block_step, ...; returns
    (out, lse or None). With want_lse the output is the fp32 partial of a KV shard. `out_buffers` = (out, lse)
    makes the kernels write into existing tensors (the slots of a gather buffer) instead of new ones."""
    lib = _lib.load()
    batch, q_heads, head_dim = query.shape
    k_cache = _rows_readable(k_cache, "the key cache of flash_attention_decode_paged")
    v_cache = _rows_readable(v_cache, "the value cache of flash_attention_decode_paged")
    if out_buffers is not None:
        out, lse = out_buffers
    else:
        out = torch.empty(query.shape, dtype=torch.float32 if out_f32 else query.dtype, device=query.device)
        lse = torch.empty((batch, q_heads), dtype=torch.float32, device=query.device) if want_lse else None
    p = _lib.PagedParams()
    p.dtype = _DTYPE_CODE[query.dtype]
    p.batch, p.heads_q, p.heads_kv, p.head_dim = batch, q_heads, k_cache.shape[2], head_dim
    p.num_blocks, p.block_size, p.max_blocks = k_cache.shape[0], k_cache.shape[1], block_table.shape[1]
    p.q, p.k_cache, p.v_cache = query.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    p.block_table, p.context_lens, p.out = block_table.data_ptr(), context_lens.data_ptr(), out.data_ptr()
    for i, s in enumerate(query.stride()):
        p.q_strides[i] = s
    _set4(p.k_strides, k_cache.stride())
    _set4(p.v_strides, v_cache.stride())
    p.bt_strides[0], p.bt_strides[1] = block_table.stride()
    p.cl_stride = context_lens.stride(0)
    for i, s in enumerate(out.stride()):
        p.o_strides[i] = s
    p.softmax_scale = float(softmax_scale)
    p.num_splits = int(num_splits)
    p.first_block, p.block_step = int(first_block), int(block_step)
    p.out_is_f32 = int(out_f32)
    p.force_path = int(force_path)
    p.status = _status_word(query.device).data_ptr()
    p.balance = int(bool(balance))
    if lse is not None:
        p.lse_out = lse.data_ptr()
    if num_splits > 1:
        o_partial = torch.empty((batch, q_heads, num_splits, head_dim), dtype=torch.float32, device=query.device)
        lse_partial = torch.empty((batch, q_heads, num_splits), dtype=torch.float32, device=query.device)
        p.o_partial, p.lse_partial = o_partial.data_ptr(), lse_partial.data_ptr()
    with torch.cuda.device(query.device):
        _lib.check(lib.fa_decode_paged(C.byref(p), _stream(query.device)))
    return out, lse


@torch.library.custom_op("fa_b200::decode_paged", mutates_args=())
def _paged_op(query: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
              context_lens: torch.Tensor, softmax_scale: float, num_splits: int, balance: bool = False) -> torch.Tensor:
    return _paged_launch(query, k_cache, v_cache, block_table, context_lens, softmax_scale, num_splits,
                         balance=balance)[0]


@_paged_op.register_fake
def _(query, k_cache, v_cache, block_table, context_lens, softmax_scale, num_splits, balance=False):
    return torch.empty_like(query)


def flash_attention_decode_paged(query, k_cache, v_cache, block_table, context_lens,
                                 softmax_scale=None, *, max_context_len=None, num_splits=None):
    """Decode attention over a paged (block-table) KV cache, vLLM style.

    query ``(batch, q_heads, head_dim)``; caches ``(num_blocks, block_size, kv_heads, head_dim)``;
    ``block_table`` int32 ``(batch, max_blocks_per_seq)``; ``context_lens`` int32 ``(batch,)``.
    ``max_context_len`` is a host-known bound used only to pick the split count (no device read-back);
    ``num_splits`` forces 1..32 splits. Non-causal, inference-only.
    Same contract as fa_rdna3/interface.py:643-728.
    """
    validate_paged_inputs(query, k_cache, v_cache, block_table, context_lens)
    validate_inference_only(query, k_cache, v_cache)
    validate_softmax_scale(softmax_scale)
    if (max_context_len is not None
            and (isinstance(max_context_len, bool) or not isinstance(max_context_len, Integral)
                 or max_context_len < 0)):
        raise ValueError("max_context_len must be a nonnegative integer or None")
    if (num_splits is not None
            and (isinstance(num_splits, bool) or not isinstance(num_splits, Integral)
                 or not 1 <= num_splits <= 32)):
        raise ValueError("num_splits must be an integer between 1 and 32 or None")
    batch, q_heads, head_dim = query.shape
    block_size = k_cache.shape[1]
    softmax_scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    balance = False
    if num_splits is not None:
        selected = int(num_splits)
    else:
        sm_count = torch.cuda.get_device_properties(query.device).multi_processor_count
        kv_heads = k_cache.shape[2]
        group = q_heads // kv_heads
        tensor_core = _paged_tensor_core_ok(query, head_dim, q_heads, kv_heads, block_size, softmax_scale)
        bound = None if max_context_len is None else int(max_context_len)
        selected = _paged_splits_b200(batch, kv_heads, group, block_size, block_table.shape[1], sm_count, bound,
                                      tensor_core=tensor_core)
        if tensor_core and selected > 1 and batch <= min(256, sm_count):
            # One CTA per SM, dealt to the sequences on the device in proportion to their context lengths (the host
            # only knows the bound): `selected` becomes the partial slots per sequence, two per CTA it may get.
            balance = True
            selected = _paged_balanced_slots(kv_heads, block_size, block_table.shape[1], sm_count, bound)
    return _paged_op(query, k_cache, v_cache, block_table, context_lens, softmax_scale, selected, balance)


# Dao-AILab style spellings of the two training entry points (same functions, same layouts as above).
flash_attn_func = flash_attention
flash_attn_varlen_func = flash_attention_varlen
