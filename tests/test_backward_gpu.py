"""Dense backward parity (dQ, dK, dV relative L2 <= 1e-2) against autograd over the fp32 oracle.

Grid modelled on the reference's tests/test_backward.py, tests/test_causal_align.py, tests/test_gqa.py,
tests/test_window.py, tests/test_softcap.py, tests/test_alibi.py, tests/test_bias.py, tests/test_dropout.py.
"""
import math

import pytest
import torch

from helpers import assert_close_grad, assert_close_o, max_abs, seeded
from oracle.attention_oracle import alibi_slopes_ref, attention_grads_ref

pytestmark = pytest.mark.gpu


def run_case(dtype, B, H, Hk, Sq, Sk, D, path="auto", seed=0, **opts):
    from fa_b200 import interface

    q = seeded(seed + 1, B, H, Sq, D, dtype=dtype)
    k = seeded(seed + 2, B, Hk, Sk, D, dtype=dtype)
    v = seeded(seed + 3, B, Hk, Sk, D, dtype=dtype)
    dout = seeded(seed + 4, B, H, Sq, D, dtype=dtype)
    scale = 1.0 / math.sqrt(D)
    causal = opts.get("causal", False)
    window = opts.get("window", (-1, -1))
    softcap = opts.get("softcap", 0.0)
    bias = opts.get("bias")
    p, dseed = opts.get("dropout_p", 0.0), opts.get("dropout_seed", 0)
    slopes = alibi_slopes_ref(H).cuda() if opts.get("alibi") else None
    with interface.force_kernel_path(path):
        out, lse = interface._forward(q, k, v, causal, scale, window, softcap, bias, slopes, p, dseed)
        dq, dk, dv = interface._backward(dout, q, k, v, out, lse, causal, scale, window, softcap, bias, slopes, p,
                                         dseed)
        used = interface.last_kernel_path()
    torch.cuda.synchronize()
    ro, rl, rdq, rdk, rdv = attention_grads_ref(
        q.cpu(), k.cpu(), v.cpu(), dout.cpu(), causal=causal, softmax_scale=scale, window=window, softcap=softcap,
        bias=None if bias is None else bias.cpu(), alibi_slopes=None if slopes is None else slopes.cpu(),
        dropout_p=p, dropout_seed=dseed)
    assert_close_o(out, ro, dtype)
    assert_close_grad(dq, rdq, "dq")
    assert_close_grad(dk, rdk, "dk")
    assert_close_grad(dv, rdv, "dv")
    return used


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("seqlen", [128, 200, 512, 1000])
def test_backward_tensor_core(dtype, causal, head_dim, seqlen):
    used = run_case(dtype, 2, 4, 4, seqlen, seqlen, head_dim, path="tcgen05", seed=seqlen + head_dim, causal=causal)
    assert used == "tcgen05"


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("head_dim", [16, 32, 256])
def test_backward_other_head_dims(causal, head_dim):
    run_case(torch.float16, 1, 2, 2, 200, 200, head_dim, seed=head_dim, causal=causal)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("sq,sk,causal", [(333, 777, False), (777, 333, False), (128, 384, True), (384, 128, True),
                                          (256, 64, True), (200, 333, True)])
def test_backward_cross_and_alignment(path, sq, sk, causal):
    run_case(torch.float16, 1, 4, 4, sq, sk, 64, path=path, seed=sq + sk, causal=causal)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("hq,hk", [(32, 8), (8, 1)])
def test_backward_gqa(path, hq, hk):
    run_case(torch.float16, 1, hq, hk, 300, 300, 64, path=path, seed=hq + hk, causal=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("window,causal,sq,sk", [((63, 0), True, 512, 512), ((48, 48), False, 400, 400),
                                                 ((31, 17), False, 96, 257), ((31, 17), False, 257, 96)])
def test_backward_window(path, window, causal, sq, sk):
    run_case(torch.float16, 1, 4, 4, sq, sk, 64, path=path, seed=window[0] + sq, causal=causal, window=window)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
def test_backward_softcap_alibi(path):
    run_case(torch.float16, 1, 8, 8, 384, 384, 128, path=path, seed=9, softcap=30.0, alibi=True, causal=True)
    run_case(torch.bfloat16, 1, 12, 12, 200, 333, 64, path=path, seed=10, softcap=50.0, alibi=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
def test_backward_bias_and_masked_rows(path):
    B, H, Sq, Sk = 2, 4, 200, 264
    g = torch.Generator().manual_seed(7)
    bias = torch.randn(1, H, Sq, Sk, generator=g)
    bias[..., 5:9, :] = float("-inf")  # fully masked rows: zero output, zero dQ
    bias[..., :, 100:140] = float("-inf")
    run_case(torch.float16, B, H, H, Sq, Sk, 64, path=path, seed=3, bias=bias.cuda())


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
def test_backward_dropout_fixed_seed(path):
    # the oracle regenerates the same Philox mask, so forward and backward masks are pinned bit for bit
    run_case(torch.float16, 2, 2, 2, 200, 264, 64, path=path, seed=5, dropout_p=0.2, dropout_seed=777)


def test_dropout_p0_is_exact_and_unbiased():
    import fa_b200

    q, k, v = (seeded(i, 1, 4, 256, 64) for i in (1, 2, 3))
    ref = fa_b200.flash_attention(q, k, v, causal=True)
    assert torch.equal(ref, fa_b200.flash_attention(q, k, v, causal=True, dropout_p=0.0))
    base = fa_b200.flash_attention(q, k, v).float()
    torch.manual_seed(1)
    acc = torch.zeros_like(base)
    n = 200
    for _ in range(n):
        acc += fa_b200.flash_attention(q, k, v, dropout_p=0.25).float()
    assert (acc / n - base).abs().mean().item() < 8e-3


def test_autograd_through_public_api():
    import fa_b200

    q, k, v = (seeded(i, 2, 4, 300, 128).requires_grad_(True) for i in (1, 2, 3))
    dout = seeded(4, 2, 4, 300, 128)
    fa_b200.flash_attention(q, k, v, causal=True).backward(dout)
    _, _, rdq, rdk, rdv = attention_grads_ref(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), dout.cpu(),
                                              causal=True)
    assert_close_grad(q.grad, rdq, "dq")
    assert_close_grad(k.grad, rdk, "dk")
    assert_close_grad(v.grad, rdv, "dv")


def test_fp32_and_padded_head_dim_gradients():
    import fa_b200

    q, k, v = (seeded(i, 1, 2, 150, 80, dtype=torch.float32).requires_grad_(True) for i in (1, 2, 3))
    dout = seeded(4, 1, 2, 150, 80, dtype=torch.float32)
    fa_b200.flash_attention(q, k, v, causal=True).backward(dout)
    assert q.grad.shape == q.shape
    _, _, rdq, rdk, rdv = attention_grads_ref(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), dout.cpu(),
                                              causal=True)
    assert_close_grad(q.grad, rdq, "dq")
    assert_close_grad(k.grad, rdk, "dk")
    assert_close_grad(v.grad, rdv, "dv")


def test_backward_run_to_run_identical():
    from fa_b200 import interface

    q, k, v, dout = (seeded(i, 1, 8, 1024, 128) for i in (1, 2, 3, 4))
    out, lse = interface._forward(q, k, v, True, 0.0884, (-1, -1), 0.0, None, None, 0.0, 0)
    a = interface._backward(dout, q, k, v, out, lse, True, 0.0884, (-1, -1), 0.0, None, None, 0.0, 0)
    b = interface._backward(dout, q, k, v, out, lse, True, 0.0884, (-1, -1), 0.0, None, None, 0.0, 0)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_backward_one_call_equals_three_calls():
    """fa_bwd with every part in one call starts dK/dV behind the delta kernel as its programmatic dependent (dK/dV CTAs
    may run before delta has finished and wait where they first read it). The gradients must be bit-identical to
    delta, dK/dV and dQ launched as three calls, each behind the completed one before it; stale delta values would
    show here. Large enough for several waves of dK/dV CTAs; with and without the dS scratch."""
    import ctypes as C

    from fa_b200 import _lib, interface

    lib = _lib.load()
    q, k, v, dout = (seeded(i, 2, 16, 2048, 128) for i in (11, 12, 13, 14))
    scale = 0.0884
    out, lse = interface._forward(q, k, v, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for scratch in (True, False):
        results = []
        for split in (False, True):
            delta = torch.full_like(lse, float("nan"))  # a read before delta is written would poison the gradients
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            p = interface._attn_params(q, k, v, out, lse, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
            interface._fill_backward(p, dout, delta, dq, dk, dv, False)
            ws = interface._ds_workspace(p, q.device) if scratch else None
            assert (ws is not None) == scratch
            for parts in ((_lib.FA_BWD_DELTA, _lib.FA_BWD_DKDV, _lib.FA_BWD_DQ) if split else (0,)):
                p.bwd_parts = parts
                _lib.check(lib.fa_bwd(C.byref(p), stream))
                if split:
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
            results.append((dq, dk, dv))
            del ws
        for one, three, name in zip(results[0], results[1], ("dq", "dk", "dv")):
            assert not torch.isnan(one).any(), name
            assert torch.equal(one, three), (name, scratch)
    import fa_b200
    fa_b200.check_status()


# ------------------------------------------------------------------------------------------------ output canaries
# compute-sanitizer is not available where these tests run, so stray writes are looked for the plain way: every
# output lives in the middle of a larger buffer that starts out as NaN. After the call the guard zones on both sides
# must still be all NaN (nothing wrote outside) and the outputs must hold no NaN (every element was written).
def _guarded(shape, dtype, guard=4096):
    n = 1
    for d in shape:
        n *= d
    buf = torch.full((n + 2 * guard,), float("nan"), dtype=dtype, device="cuda")
    return buf, buf[guard:guard + n].view(*shape), guard


def _assert_guards_intact(buf, view, guard, what):
    assert torch.isnan(buf[:guard]).all() and torch.isnan(buf[guard + view.numel():]).all(), f"{what}: guard zone written"
    assert not torch.isnan(view.float()).any(), f"{what}: an element was left unwritten"


@pytest.mark.parametrize("path", [1, 2])  # tensor-core kernels, CUDA-core kernels
@pytest.mark.parametrize("B,H,Hk,Sq,Sk,D,causal", [(2, 4, 2, 200, 333, 128, False), (1, 3, 3, 257, 257, 64, True),
                                                   (1, 2, 1, 130, 77, 80, True)])
def test_forward_backward_write_exactly_their_outputs(path, B, H, Hk, Sq, Sk, D, causal):
    import ctypes as C

    import fa_b200
    from fa_b200 import _lib, interface

    lib = _lib.load()
    q, k, v, dout = seeded(1, B, H, Sq, D), seeded(2, B, Hk, Sk, D), seeded(3, B, Hk, Sk, D), seeded(4, B, H, Sq, D)
    bufs = {"out": _guarded((B, H, Sq, D), torch.float16), "lse": _guarded((B, H, Sq), torch.float32),
            "delta": _guarded((B, H, Sq), torch.float32), "dq": _guarded((B, H, Sq, D), torch.float16),
            "dk": _guarded((B, Hk, Sk, D), torch.float16), "dv": _guarded((B, Hk, Sk, D), torch.float16)}
    t = {name: b[1] for name, b in bufs.items()}
    p = interface._attn_params(q, k, v, t["out"], t["lse"], causal, 1 / math.sqrt(D), (-1, -1), 0.0, None, None, 0.0, 0,
                               force_path=path)
    interface._fill_backward(p, dout, t["delta"], t["dq"], t["dk"], t["dv"], False)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.fa_fwd(C.byref(p), stream))
    _lib.check(lib.fa_bwd(C.byref(p), stream))
    torch.cuda.synchronize()
    assert lib.fa_last_path() == path
    for name, (buf, view, guard) in bufs.items():
        _assert_guards_intact(buf, view, guard, name)
    fa_b200.check_status()


# ------------------------------------------------------------------------------------------------ dS workspace form
@pytest.mark.parametrize("dtype,B,H,Hk,Sq,Sk,D,opts", [
    (torch.float16, 2, 4, 4, 512, 512, 128, dict(causal=True)),
    (torch.bfloat16, 1, 8, 2, 300, 700, 64, dict(causal=True)),
    (torch.float16, 1, 4, 4, 700, 300, 128, dict(causal=True)),
    (torch.float16, 1, 4, 2, 640, 640, 128, dict(causal=True, window=(100, 0))),
    (torch.float16, 1, 4, 4, 400, 400, 80, dict(window=(48, 48))),
    (torch.float16, 1, 2, 2, 384, 384, 128, dict(causal=True, softcap=30.0, alibi=True)),
    (torch.float16, 1, 2, 2, 256, 256, 64, dict(dropout_p=0.2, dropout_seed=7)),
])
def test_backward_with_and_without_ds_workspace(dtype, B, H, Hk, Sq, Sk, D, opts, monkeypatch):
    """dQ from the stored dS tiles (one GEMM) and dQ from the recomputing kernel both agree with the oracle; the
    workspace starts out as NaN, so a tile read before it was written would show."""
    from fa_b200 import interface

    monkeypatch.setattr(interface, "_poison_ds_workspace", True)
    for limit in (1 << 30, 0):
        monkeypatch.setattr(interface, "DS_WORKSPACE_LIMIT_BYTES", limit)
        assert run_case(dtype, B, H, Hk, Sq, Sk, D, path="tcgen05", **opts) == "tcgen05"


# ------------------------------------------------------------------------------------- head dims above 128 (to 256)
def _bias_with_masked_rows(H, Sq, Sk):
    g = torch.Generator().manual_seed(11)
    bias = torch.randn(1, H, Sq, Sk, generator=g)
    bias[..., 5:9, :] = float("-inf")
    bias[..., :, 100:140] = float("-inf")
    return bias.cuda()


@pytest.mark.parametrize("dtype,B,H,Hk,Sq,Sk,D,opts", [
    (torch.float16, 2, 4, 4, 512, 512, 256, dict(causal=True)),
    (torch.bfloat16, 2, 4, 4, 512, 512, 256, dict()),
    (torch.float16, 1, 2, 2, 128, 128, 256, dict(causal=True)),
    (torch.float16, 1, 3, 3, 200, 200, 160, dict(causal=True)),
    (torch.bfloat16, 1, 8, 2, 300, 700, 192, dict(causal=True)),
    (torch.float16, 1, 4, 1, 700, 300, 256, dict(causal=True)),
    (torch.float16, 1, 2, 2, 77, 1000, 256, dict()),
    (torch.float16, 1, 4, 2, 640, 640, 256, dict(causal=True, window=(100, 0))),
    (torch.float16, 1, 4, 4, 400, 400, 136, dict(window=(48, 48))),
    (torch.float16, 1, 2, 2, 384, 384, 256, dict(causal=True, softcap=30.0, alibi=True)),
    (torch.bfloat16, 1, 4, 4, 200, 333, 224, dict(softcap=50.0, alibi=True)),
    (torch.float16, 2, 2, 2, 256, 264, 256, dict(dropout_p=0.2, dropout_seed=7)),
    (torch.float16, 2, 4, 4, 200, 264, 256, dict(bias="masked_rows")),
])
def test_backward_wide_head_dims_on_tensor_cores(dtype, B, H, Hk, Sq, Sk, D, opts, monkeypatch):
    """Head dims in (128, 256]: scores kernel + three products over the P / dS tiles. The workspace starts out as NaN,
    so a tile that is read without having been written would show."""
    from fa_b200 import interface

    opts = dict(opts)
    if opts.get("bias") == "masked_rows":
        opts["bias"] = _bias_with_masked_rows(H, Sq, Sk)
    monkeypatch.setattr(interface, "_poison_ds_workspace", True)
    assert run_case(dtype, B, H, Hk, Sq, Sk, D, path="tcgen05", seed=Sq + D, **opts) == "tcgen05"


def test_backward_wide_in_batch_pieces_matches_one_launch(monkeypatch):
    """A batch whose scratch exceeds the limit is taken entry by entry; gradients are bit-identical to one launch."""
    from fa_b200 import interface

    B, H, S, D = 3, 2, 256, 256
    q, k, v, dout = (seeded(40 + i, B, H, S, D) for i in range(4))
    scale = 1.0 / math.sqrt(D)
    out, lse = interface._forward(q, k, v, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    with interface.force_kernel_path("tcgen05"):
        whole = interface._backward(dout, q, k, v, out, lse, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
        per_entry = 2 * H * 2 * 2 * 32768
        monkeypatch.setattr(interface, "DS_WORKSPACE_WIDE_LIMIT_BYTES", per_entry)
        assert interface._wide_batch_pieces(q, k, 2, 128) == [(0, 1), (1, 2), (2, 3)]
        pieces = interface._backward(dout, q, k, v, out, lse, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    for a, b in zip(whole, pieces):
        assert torch.equal(a, b)


def test_backward_wide_without_scratch_falls_to_cuda_cores(monkeypatch):
    from fa_b200 import interface

    monkeypatch.setattr(interface, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 0)
    assert run_case(torch.float16, 1, 2, 2, 200, 200, 256, seed=3, causal=True) == "simt"


# ------------------------------------------------------------------------------------- head dims above 256 (to 512)
@pytest.mark.parametrize("dtype,B,H,Hk,Sq,Sk,D,opts", [
    (torch.float16, 2, 2, 2, 512, 512, 512, dict(causal=True)),
    (torch.bfloat16, 1, 4, 4, 384, 384, 512, dict()),
    (torch.float16, 1, 3, 3, 200, 200, 320, dict(causal=True)),
    (torch.bfloat16, 1, 8, 2, 300, 700, 384, dict(causal=True)),
    (torch.float16, 1, 4, 1, 700, 300, 512, dict(causal=True)),
    (torch.float16, 1, 2, 2, 77, 1000, 264, dict()),
    (torch.float16, 1, 4, 2, 640, 640, 448, dict(causal=True, window=(100, 0))),
])
def test_backward_very_wide_head_dims_on_tensor_cores(dtype, B, H, Hk, Sq, Sk, D, opts, monkeypatch):
    """Head dims in (256, 512] without score modifiers: P tiles, dS tiles (P read back from its tile), then the three
    products once per 256 columns. The scratch starts out as NaN."""
    from fa_b200 import interface

    monkeypatch.setattr(interface, "_poison_ds_workspace", True)
    assert run_case(dtype, B, H, Hk, Sq, Sk, D, path="tcgen05", seed=Sq + D, **opts) == "tcgen05"


def test_backward_very_wide_with_modifiers_runs_on_cuda_cores():
    assert run_case(torch.float16, 1, 2, 2, 200, 200, 512, seed=4, causal=True, softcap=20.0) == "simt"
