"""ctypes binding of libfa_b200.so, the C-ABI CUDA library declared in include/fa_b200.h.

The structures below mirror the header field for field. Loading is lazy and loud: there is no CPU or
PyTorch fallback, so a missing library raises instead of silently degrading.
"""
import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfa_b200.so")

FA_F16, FA_BF16, FA_F32 = 0, 1, 2
FA_PATH_NONE, FA_PATH_TCGEN05, FA_PATH_SIMT = 0, 1, 2
FA_BWD_DELTA, FA_BWD_DKDV, FA_BWD_DQ = 1, 2, 4
FA_WS_BWD_DELTA, FA_WS_DECODE_O_PARTIAL, FA_WS_DECODE_LSE_PARTIAL, FA_WS_PAGED_O_PARTIAL, FA_WS_PAGED_LSE_PARTIAL = 1, 2, 3, 4, 5
FA_WS_BWD_DS = 6
FA_WS_FWD_P = 7
ABI_VERSION = 3

I64x4 = C.c_int64 * 4
I64x3 = C.c_int64 * 3
I64x2 = C.c_int64 * 2


class AttnParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("varlen", C.c_int32),
        ("batch", C.c_int32), ("heads_q", C.c_int32), ("heads_kv", C.c_int32),
        ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32), ("head_dim", C.c_int32),
        ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("q", C.c_void_p), ("q_strides", I64x4),
        ("k", C.c_void_p), ("k_strides", I64x4),
        ("v", C.c_void_p), ("v_strides", I64x4),
        ("out", C.c_void_p), ("o_strides", I64x4),
        ("lse", C.c_void_p), ("lse_strides", I64x3),
        ("dout", C.c_void_p), ("do_strides", I64x4),
        ("delta", C.c_void_p), ("delta_strides", I64x3),
        ("dq", C.c_void_p), ("dq_strides", I64x4),
        ("dk", C.c_void_p), ("dk_strides", I64x4),
        ("dv", C.c_void_p), ("dv_strides", I64x4),
        ("softmax_scale", C.c_float), ("softcap", C.c_float),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int32), ("bias_strides", I64x4),
        ("alibi_slopes", C.c_void_p),
        ("causal", C.c_int32), ("window_left", C.c_int32), ("window_right", C.c_int32),
        ("dropout_p", C.c_float), ("dropout_seed", C.c_uint64),
        ("status", C.c_void_p), ("force_path", C.c_int32), ("bwd_parts", C.c_int32),
        ("ds_workspace", C.c_void_p), ("ds_workspace_bytes", C.c_int64),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("heads_q", C.c_int32), ("heads_kv", C.c_int32),
        ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32), ("head_dim", C.c_int32),
        ("q", C.c_void_p), ("q_strides", I64x4),
        ("k", C.c_void_p), ("k_strides", I64x4),
        ("v", C.c_void_p), ("v_strides", I64x4),
        ("out", C.c_void_p), ("o_strides", I64x4),
        ("softmax_scale", C.c_float), ("num_splits", C.c_int32),
        ("o_partial", C.c_void_p), ("lse_partial", C.c_void_p), ("force_path", C.c_int32),
        ("status", C.c_void_p),
    ]


class CombineParams(C.Structure):
    _fields_ = [
        ("out_dtype", C.c_int32), ("rows", C.c_int32), ("head_dim", C.c_int32), ("num_splits", C.c_int32),
        ("o_partial", C.c_void_p), ("o_split_stride", C.c_int64), ("o_row_stride", C.c_int64),
        ("lse_partial", C.c_void_p), ("lse_split_stride", C.c_int64), ("lse_row_stride", C.c_int64),
        ("out", C.c_void_p), ("out_row_stride", C.c_int64),
        ("lse_out", C.c_void_p),
    ]


FA_MAX_PEERS = 16


class PeerMergeParams(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32),
        ("out_dtype", C.c_int32), ("rows", C.c_int32), ("head_dim", C.c_int32),
        ("epoch", C.c_int32),
        ("slot_floats", C.c_int64),
        ("peer_base", C.c_void_p * FA_MAX_PEERS),
        ("peer_flags", C.c_void_p * FA_MAX_PEERS),
        ("out", C.c_void_p), ("out_row_stride", C.c_int64),
        ("lse_out", C.c_void_p),
        ("status", C.c_void_p),
    ]


class PagedParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("heads_q", C.c_int32), ("heads_kv", C.c_int32), ("head_dim", C.c_int32),
        ("num_blocks", C.c_int32), ("block_size", C.c_int32), ("max_blocks", C.c_int32),
        ("q", C.c_void_p), ("q_strides", I64x3),
        ("k_cache", C.c_void_p), ("k_strides", I64x4),
        ("v_cache", C.c_void_p), ("v_strides", I64x4),
        ("block_table", C.c_void_p), ("bt_strides", I64x2),
        ("context_lens", C.c_void_p), ("cl_stride", C.c_int64),
        ("out", C.c_void_p), ("o_strides", I64x3),
        ("softmax_scale", C.c_float), ("num_splits", C.c_int32),
        ("first_block", C.c_int32), ("block_step", C.c_int32),
        ("o_partial", C.c_void_p), ("lse_partial", C.c_void_p), ("lse_out", C.c_void_p),
        ("out_is_f32", C.c_int32), ("force_path", C.c_int32),
        ("status", C.c_void_p), ("balance", C.c_int32),
    ]


class TinyParams(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("heads", C.c_int32), ("seqlen", C.c_int32), ("head_dim", C.c_int32),
        ("q", C.c_void_p), ("q_strides", I64x4),
        ("k", C.c_void_p), ("k_strides", I64x4),
        ("v", C.c_void_p), ("v_strides", I64x4),
        ("out", C.c_void_p), ("o_strides", I64x4),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int32), ("bias_strides", I64x4),
        ("softmax_scale", C.c_float),
    ]


# name -> (restype, argtypes); the symbol list that include/fa_b200.h declares
SYMBOLS = {
    "fa_abi_version": (C.c_int32, []),
    "fa_device_supported": (C.c_int32, [C.c_int32]),
    "fa_last_error_string": (C.c_char_p, []),
    "fa_last_path": (C.c_int32, []),
    "fa_fwd": (C.c_int32, [C.POINTER(AttnParams), C.c_void_p]),
    "fa_bwd_delta": (C.c_int32, [C.POINTER(AttnParams), C.c_void_p]),
    "fa_bwd": (C.c_int32, [C.POINTER(AttnParams), C.c_void_p]),
    "fa_varlen_fwd": (C.c_int32, [C.POINTER(AttnParams), C.c_void_p]),
    "fa_varlen_bwd": (C.c_int32, [C.POINTER(AttnParams), C.c_void_p]),
    "fa_decode_splitk": (C.c_int32, [C.POINTER(DecodeParams), C.c_void_p]),
    "fa_decode_splitk_noalloc": (C.c_int32, [C.POINTER(DecodeParams), C.c_void_p]),
    "fa_combine": (C.c_int32, [C.POINTER(CombineParams), C.c_void_p]),
    "fa_decode_paged": (C.c_int32, [C.POINTER(PagedParams), C.c_void_p]),
    "fa_tiny_fwd": (C.c_int32, [C.POINTER(TinyParams), C.c_void_p]),
    "fa_workspace_bytes": (C.c_int64, [C.c_int32, C.c_void_p]),
    "fa_test_decode_fault": (None, [C.c_uint32, C.c_int32]),
    "fa_peer_merge": (C.c_int32, [C.POINTER(PeerMergeParams), C.c_void_p]),
    "fa_enable_peer_access": (C.c_int32, [C.c_int32]),
}

_lib = None
_lock = threading.Lock()


def load():
    """Return the loaded library; raise RuntimeError with build instructions if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"fa_b200: {LIB_PATH} is missing; build it with "
                    "`python flash-attention-rdna3_b200/build.py` (there is no fallback path)")
            lib = C.CDLL(LIB_PATH)
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            if lib.fa_abi_version() != ABI_VERSION:
                raise RuntimeError(f"fa_b200: {LIB_PATH} has ABI version {lib.fa_abi_version()}, this package expects "
                                   f"{ABI_VERSION}; rebuild it with `python flash-attention-rdna3_b200/build.py`")
            _lib = lib
    return _lib


def check(rc):
    """Turn a non-zero status of a C call into RuntimeError carrying the library's message."""
    if rc != 0:
        msg = load().fa_last_error_string()
        raise RuntimeError(f"fa_b200 error {rc}: {msg.decode() if msg else 'unknown'}")
