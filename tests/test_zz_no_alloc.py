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
import os
import subprocess
import sys

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


_FRESH_PROCESS = r"""
import ctypes as C, math, sys, torch
sys.path[:0] = {paths!r}
from fa_b200 import _lib
from helpers import seeded, max_abs, O_TOL
sys.path.insert(0, {tests!r})
import test_zz_no_alloc as t
lib = _lib.load()
torch.cuda.init()
# The library's copy of the CUDA runtime attaches to the context on its first call and, with eager module loading,
# loads the library's code and fixed arrays then; that is done here, by a query that launches nothing.
assert lib.fa_device_supported(0) == 0
stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
# 1 row x 128 dims x 8 partials per kv head: the tensor-core kernel with the merge (and its ticket words) inside
q, k, v = seeded(11, 2, 8, 1, 128), seeded(12, 2, 8, 4096, 128), seeded(13, 2, 8, 4096, 128)
got, want = torch.empty_like(q), torch.empty_like(q)
o_partial = torch.empty(8, 2, 8, 1, 128, dtype=torch.float32, device="cuda")
lse_partial = torch.empty(8, 2, 8, 1, dtype=torch.float32, device="cuda")
p = t._params(q, k, v, got, 8)
torch.cuda.synchronize()
free_before = torch.cuda.mem_get_info()[0]
_lib.check(lib.fa_decode_splitk_noalloc(C.byref(p), stream))   # the first launch this process makes in the library
torch.cuda.synchronize()
free_after = torch.cuda.mem_get_info()[0]
assert lib.fa_last_path() == _lib.FA_PATH_TCGEN05
_lib.check(lib.fa_decode_splitk(C.byref(t._params(q, k, v, want, 8, o_partial, lse_partial)), stream))
torch.cuda.synchronize()
assert max_abs(got, want) <= O_TOL[torch.float16], max_abs(got, want)
print("FREE", free_before, free_after)
"""


def test_first_call_of_a_process_takes_no_device_memory():
    """A fresh process whose very first launch in the library is the no-allocation entry point, on a shape that
    runs the tensor-core kernel with the merge inside (the path that uses the library's ticket words): the device's
    free memory (cudaMemGetInfo, which sees every allocation of the process, torch's or not) must be the same before
    and after. All modules are loaded eagerly so that loading code does not count as allocating."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _FRESH_PROCESS.format(paths=[root, os.path.join(root, "flash-attention-rdna3_b200"),
                                        os.path.join(root, "tests")], tests=os.path.join(root, "tests"))
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    before, after = (int(x) for x in r.stdout.split("FREE")[1].split())
    assert after == before, f"free device memory went from {before} to {after} bytes across the call"


def test_largest_accepted_and_smallest_refused_problem():
    """The limit is num_splits * rows * (head_dim + 1) <= 2 Mi floats: 16 x 1016 x 129 fits, 16 x 1024 x 129 does not."""
    from fa_b200 import _lib

    lib = _lib.load()
    _run_pair(31, 127, 8, 1, 1, 2048, 128, 16)
    q, k = seeded(1, 128, 8, 1, 128), seeded(2, 128, 1, 256, 128)
    p = _params(q, k, k, torch.empty_like(q), 16)
    rc = lib.fa_decode_splitk_noalloc(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2


def test_oversized_problem_is_refused():
    from fa_b200 import _lib

    lib = _lib.load()
    q, k = seeded(1, 64, 64, 8, 128), seeded(2, 64, 64, 64, 128)
    out = torch.empty_like(q)
    p = _params(q, k, k, out, 64)  # 64 * 64*64*8 * 129 floats > 2 Mi
    rc = lib.fa_decode_splitk_noalloc(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2
    assert b"exceeds the built-in scratch" in lib.fa_last_error_string()
