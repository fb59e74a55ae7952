"""Dense forward parity against the fp32 oracle, through the public API and the C ABI.

Grid modelled on the reference's tests/test_forward.py, tests/test_causal_align.py, tests/test_gqa.py,
tests/test_window.py, tests/test_softcap.py, tests/test_alibi.py, tests/test_bias.py.
"""
import math

import pytest
import torch

from helpers import assert_close_o, max_abs, seeded
from oracle.attention_oracle import alibi_slopes_ref, attention_ref

pytestmark = pytest.mark.gpu


def run_case(dtype, B, H, Hk, Sq, Sk, D, path="auto", seed=0, **opts):
    import fa_b200
    from fa_b200 import interface

    q = seeded(seed + 1, B, H, Sq, D, dtype=dtype)
    k = seeded(seed + 2, B, Hk, Sk, D, dtype=dtype)
    v = seeded(seed + 3, B, Hk, Sk, D, dtype=dtype)
    scale = 1.0 / math.sqrt(D)
    causal = opts.get("causal", False)
    window = opts.get("window", (-1, -1))
    softcap = opts.get("softcap", 0.0)
    bias = opts.get("bias")
    slopes = alibi_slopes_ref(H).cuda() if opts.get("alibi") else None
    with interface.force_kernel_path(path):
        out, lse = interface._forward(q, k, v, causal, scale, window, softcap, bias, slopes, 0.0, 0)
        used = interface.last_kernel_path()
    torch.cuda.synchronize()
    ref_o, ref_l = attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=causal, softmax_scale=scale, window=window,
                                 softcap=softcap, bias=None if bias is None else bias.cpu(),
                                 alibi_slopes=None if slopes is None else slopes.cpu())
    assert_close_o(out, ref_o, dtype)
    assert_close_o(lse, ref_l, dtype, "lse")
    return used


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("seqlen", [128, 200, 512, 1000, 2048])
def test_forward_tensor_core(dtype, causal, head_dim, seqlen):
    used = run_case(dtype, 2, 4, 4, seqlen, seqlen, head_dim, path="tcgen05", seed=seqlen + head_dim, causal=causal)
    assert used == "tcgen05"


@pytest.mark.parametrize("head_dim", [16, 32, 64, 128, 256])
def test_forward_head_dims(head_dim):
    run_case(torch.float16, 1, 2, 2, 300, 300, head_dim, seed=head_dim)


def test_forward_single_token():
    run_case(torch.float16, 1, 1, 1, 1, 1, 64, seed=5)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("sq,sk", [(333, 777), (777, 333), (1, 500), (129, 1)])
def test_forward_cross_attention(path, sq, sk):
    run_case(torch.float16, 2, 4, 4, sq, sk, 64, path=path, seed=sq + sk)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("sq,sk", [(128, 384), (384, 128), (256, 64), (200, 333)])
def test_forward_causal_bottom_right(path, sq, sk):
    # Sq > Sk leaves the first rows without any visible key: O = 0, LSE = -inf
    run_case(torch.float16, 1, 4, 4, sq, sk, 64, path=path, seed=sq * 3 + sk, causal=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("hq,hk", [(32, 8), (16, 4), (8, 1)])
def test_forward_gqa(path, hq, hk):
    run_case(torch.float16, 1, hq, hk, 300, 300, 64, path=path, seed=hq + hk, causal=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("window,causal,sq,sk", [((63, 0), True, 512, 512), ((255, 0), True, 700, 700),
                                                 ((48, 48), False, 400, 400), ((100, 0), False, 300, 300),
                                                 ((31, 17), False, 96, 257), ((31, 17), False, 257, 96)])
def test_forward_window(path, window, causal, sq, sk):
    run_case(torch.float16, 1, 4, 4, sq, sk, 64, path=path, seed=window[0] + sq, causal=causal, window=window)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("softcap", [30.0, 50.0])
def test_forward_softcap(path, softcap):
    run_case(torch.float16, 1, 4, 4, 384, 384, 128, path=path, seed=int(softcap), softcap=softcap, causal=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("heads", [8, 12])
def test_forward_alibi(path, heads):
    run_case(torch.float16, 1, heads, heads, 300, 420, 64, path=path, seed=heads, alibi=True, causal=True)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("kind", ["full", "batch_broadcast", "head_broadcast", "hard_mask", "all_masked_rows"])
def test_forward_bias(path, kind):
    B, H, Sq, Sk = 2, 4, 200, 264
    g = torch.Generator().manual_seed(7)
    shape = {"full": (B, H, Sq, Sk), "batch_broadcast": (1, H, Sq, Sk), "head_broadcast": (B, 1, Sq, Sk),
             "hard_mask": (1, 1, Sq, Sk), "all_masked_rows": (1, 1, Sq, Sk)}[kind]
    bias = torch.randn(shape, generator=g)
    if kind == "hard_mask":
        bias = torch.where(torch.rand(shape, generator=g) < 0.3, torch.full(shape, float("-inf")), bias)
    if kind == "all_masked_rows":
        bias[..., 5:9, :] = float("-inf")          # rows with no visible key at all
        bias[..., 40:60, :130] = float("-inf")     # a whole 128-key tile masked, then very negative logits
        bias[..., 40:60, 130:] -= 1000.0
    run_case(torch.float16, B, H, H, Sq, Sk, 64, path=path, seed=3, bias=bias.cuda())


def test_forward_fp32_and_transposed_layout():
    import fa_b200

    q = seeded(1, 2, 300, 4, 64, dtype=torch.float32).transpose(1, 2)   # (B, H, S, D) view of (B, S, H, D)
    k = seeded(2, 2, 300, 4, 64, dtype=torch.float32).transpose(1, 2)
    v = seeded(3, 2, 300, 4, 64, dtype=torch.float32).transpose(1, 2)
    out = fa_b200.flash_attention(q, k, v, causal=True)
    ref, _ = attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert max_abs(out, ref) <= 2e-3


def test_forward_transposed_layout_stays_on_tensor_cores():
    from fa_b200 import interface
    import fa_b200

    q = seeded(1, 2, 384, 4, 128).transpose(1, 2)
    k = seeded(2, 2, 384, 4, 128).transpose(1, 2)
    v = seeded(3, 2, 384, 4, 128).transpose(1, 2)
    out = fa_b200.flash_attention(q, k, v)
    assert interface.last_kernel_path() == "tcgen05"
    ref, _ = attention_ref(q.cpu(), k.cpu(), v.cpu())
    assert_close_o(out, ref, torch.float16)


@pytest.mark.parametrize("head_dim", [48, 80, 96, 192])
def test_forward_padded_head_dim(head_dim):
    import fa_b200

    q, k, v = (seeded(i, 1, 2, 150, head_dim) for i in (1, 2, 3))
    out = fa_b200.flash_attention(q, k, v, causal=True)
    assert out.shape == q.shape
    ref, _ = attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert_close_o(out, ref, torch.float16)


def test_forward_run_to_run_identical():
    import fa_b200

    q, k, v = (seeded(i, 2, 8, 1024, 128) for i in (1, 2, 3))
    a = fa_b200.flash_attention(q, k, v, causal=True)
    b = fa_b200.flash_attention(q, k, v, causal=True)
    assert torch.equal(a, b)


def test_forward_matches_between_kernel_families():
    from fa_b200 import interface

    q, k, v = (seeded(i, 1, 4, 640, 128) for i in (1, 2, 3))
    with interface.force_kernel_path("tcgen05"):
        a, la = interface._forward(q, k, v, True, 0.0884, (-1, -1), 0.0, None, None, 0.0, 0)
    with interface.force_kernel_path("simt"):
        b, lb = interface._forward(q, k, v, True, 0.0884, (-1, -1), 0.0, None, None, 0.0, 0)
    assert max_abs(a, b) <= 2e-3 and max_abs(la, lb) <= 2e-3


# ------------------------------------------------------------------------------------- head dims above 256 (to 512)
@pytest.mark.parametrize("dtype,B,H,Hk,Sq,Sk,D,opts", [
    (torch.float16, 2, 2, 2, 512, 512, 512, dict()),
    (torch.bfloat16, 1, 4, 4, 512, 512, 512, dict(causal=True)),
    (torch.float16, 1, 1, 1, 128, 128, 512, dict(causal=True)),
    (torch.float16, 1, 3, 3, 200, 200, 320, dict(causal=True)),
    (torch.bfloat16, 1, 8, 2, 300, 700, 384, dict(causal=True)),
    (torch.float16, 1, 4, 1, 700, 300, 512, dict(causal=True)),      # the first 400 rows see no key
    (torch.float16, 1, 2, 2, 77, 1000, 264, dict()),
    (torch.float16, 1, 2, 2, 1, 333, 512, dict()),
    (torch.float16, 1, 4, 2, 640, 640, 448, dict(causal=True, window=(100, 0))),
    (torch.float16, 1, 2, 2, 400, 400, 512, dict(window=(48, 48))),
])
def test_forward_very_wide_head_dims_on_tensor_cores(dtype, B, H, Hk, Sq, Sk, D, opts, monkeypatch):
    """Head dims in (256, 512] without score modifiers: row statistics, normalised P tiles in a scratch buffer (poisoned
    with NaN here, so a tile read without having been written would show), O = P V as a product over those tiles."""
    from fa_b200 import interface

    monkeypatch.setattr(interface, "_poison_ds_workspace", True)
    assert run_case(dtype, B, H, Hk, Sq, Sk, D, path="tcgen05", seed=Sq + D, **opts) == "tcgen05"


def test_forward_very_wide_with_modifiers_or_without_scratch_runs_on_cuda_cores(monkeypatch):
    from fa_b200 import interface

    assert run_case(torch.float16, 1, 2, 2, 200, 200, 512, seed=1, softcap=20.0) == "simt"
    monkeypatch.setattr(interface, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 0)
    assert run_case(torch.float16, 1, 2, 2, 200, 200, 512, seed=2, causal=True) == "simt"


def test_forward_very_wide_in_batch_pieces_matches_one_launch(monkeypatch):
    from fa_b200 import interface

    B, H, S, D = 3, 2, 256, 512
    q, k, v = (seeded(60 + i, B, H, S, D) for i in range(3))
    scale = 1.0 / math.sqrt(D)
    whole = interface._forward(q, k, v, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    monkeypatch.setattr(interface, "DS_WORKSPACE_WIDE_LIMIT_BYTES", H * (2 * 2 * 32768 + 2 * 1024))
    assert interface._wide_batch_pieces(q, k, 1, 256) == [(0, 1), (1, 2), (2, 3)]
    pieces = interface._forward(q, k, v, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    assert torch.equal(whole[0], pieces[0]) and torch.equal(whole[1], pieces[1])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("pattern", ["rising", "sawtooth"])
def test_forward_running_maximum_keeps_growing(causal, head_dim, pattern):
    """Scores that rise along the keys, so that the running maximum of every row grows by more than the rescale
    threshold in (almost) every key tile (`rising`), or in every other one (`sawtooth`): the softmax path that
    exponentiates against the old maximum and redoes the tile when the maximum grew is taken tile after tile, next to
    tiles where it is not. Forward and, through the LSE it hands on, the backward must still match the oracle."""
    from fa_b200 import interface

    S, H = 1024, 2
    g = torch.Generator().manual_seed(head_dim + (1 if causal else 0))
    u = torch.ones(head_dim) / math.sqrt(head_dim)
    steps = torch.arange(S, dtype=torch.float32)
    if pattern == "sawtooth":
        steps = torch.where((steps // 128) % 2 == 0, steps, steps - 128.0)
    q = (u * 1.5 + 0.05 * torch.randn(1, H, S, head_dim, generator=g)).to(torch.float16).cuda()
    k = (u * steps[None, None, :, None] * 1.0 + 0.05 * torch.randn(1, H, S, head_dim, generator=g))
    k = k.to(torch.float16).cuda()
    v = torch.randn(1, H, S, head_dim, generator=g).to(torch.float16).cuda()
    scale = 1.0 / math.sqrt(head_dim)
    with interface.force_kernel_path("tcgen05"):
        out, lse = interface._forward(q, k, v, causal, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    torch.cuda.synchronize()
    ref_o, ref_l = attention_ref(q.cpu(), k.cpu(), v.cpu(), causal=causal, softmax_scale=scale)
    assert_close_o(out, ref_o, torch.float16)
    assert_close_o(lse, ref_l, torch.float16, "lse")
