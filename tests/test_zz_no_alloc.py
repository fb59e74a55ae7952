"""Split-K decode through the entry point that allocates nothing (fa_decode_splitk_noalloc).

Who needs it: callers that are not allowed to allocate device memory where they run attention - code inside
a serving engine's pre-sized arena, plug-ins that only get input and output buffers, latency-critical loops.
The partials live in an array built into the library, shared by every call on the device, so this test makes
two different calls in a row and checks each against the ordinary entry point (caller-provided scratch) on the
same inputs, and checks that an oversized problem is refused with a clear message.

The file name sorts last on purpose: a run that stops at the first failure has already run every other test.
"""
import ctypes as C
import math

import pytest
import torch

from helpers import O_TOL, max_abs, seeded

pytestmark = pytest.mark.gpu


def _params(q, k, v, out, splits, o_partial=None, lse_partial=None):
    from fa_b200 import _lib

    p = _lib.DecodeParams()
    p.dtype = _lib.FA_F16
    p.batch, p.heads_q, p.seqlen_q, p.head_dim = q.shape
    p.heads_kv, p.seqlen_k = k.shape[1], k.shape[2]
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    for field, t in ((p.q_strides, q), (p.k_strides, k), (p.v_strides, v), (p.o_strides, out)):
        for i, s in enumerate(t.stride()):
            field[i] = s
    p.softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    p.num_splits = splits
    if o_partial is not None:
        p.o_partial, p.lse_partial = o_partial.data_ptr(), lse_partial.data_ptr()
    return p


def _run_pair(seed, B, Hq, Hk, Sq, Sk, D, splits):
    from fa_b200 import _lib

    lib = _lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    q, k, v = seeded(seed, B, Hq, Sq, D), seeded(seed + 1, B, Hk, Sk, D), seeded(seed + 2, B, Hk, Sk, D)
    want, got = torch.empty_like(q), torch.empty_like(q)
    o_partial = torch.empty(splits, B, Hq, Sq, D, dtype=torch.float32, device="cuda")
    lse_partial = torch.empty(splits, B, Hq, Sq, dtype=torch.float32, device="cuda")
    _lib.check(lib.fa_decode_splitk(C.byref(_params(q, k, v, want, splits, o_partial, lse_partial)), stream))
    # no torch allocation happens between here and the end of the call under test
    p = _params(q, k, v, got, splits)
    before = torch.cuda.memory_allocated()
    _lib.check(lib.fa_decode_splitk_noalloc(C.byref(p), stream))
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    assert max_abs(got, want) <= O_TOL[torch.float16]
    assert not torch.isnan(got.float()).any()


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # different shapes and split counts, so the second call reuses the built-in array with another layout
    _run_pair(11, 2, 8, 8, 1, 4096, 128, 8)
    _run_pair(23, 1, 16, 4, 3, 1000, 64, 5)


def test_oversized_problem_is_refused():
    from fa_b200 import _lib

    lib = _lib.load()
    q, k = seeded(1, 64, 64, 8, 128), seeded(2, 64, 64, 64, 128)
    out = torch.empty_like(q)
    p = _params(q, k, k, out, 64)  # 64 * 64*64*8 * 129 floats > 2 Mi
    rc = lib.fa_decode_splitk_noalloc(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2
    assert b"exceeds the built-in scratch" in lib.fa_last_error_string()
