"""The CUDA kernels against the reference's own kernel outputs (tests/golden/*.npz), both kernel families."""
import math

import pytest
import torch

from golden_io import DENSE_CASES, dense_kwargs, load
from helpers import max_abs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", ["auto", "simt"])
@pytest.mark.parametrize("name", DENSE_CASES)
def test_dense_golden(name, path):
    from fa_b200 import interface

    g = load(name)
    kw = dense_kwargs(g)
    q, k, v, dout = (g[n].to(torch.float16).cuda() for n in ("q", "k", "v", "dout"))
    bias = None if kw["bias"] is None else kw["bias"].cuda()
    alibi = None if kw["alibi_slopes"] is None else kw["alibi_slopes"].cuda()
    args = (kw["causal"], kw["softmax_scale"], kw["window"], kw["softcap"], bias, alibi, kw["dropout_p"],
            kw["dropout_seed"])
    with interface.force_kernel_path(path):
        out, lse = interface._forward(q, k, v, *args)
        dq, dk, dv = interface._backward(dout, q, k, v, out, lse, *args)
    assert max_abs(out, g["out"]) <= 3e-3
    assert max_abs(lse, g["lse"]) <= 3e-3
    assert rel_l2(dq, g["dq"]) <= 1e-2 and rel_l2(dk, g["dk"]) <= 1e-2 and rel_l2(dv, g["dv"]) <= 1e-2


def test_dense_golden_head_dim_64_tensor_core():
    """The goldens use head_dim 32 (CUDA-core family); zero-padding to 64 runs them on the tcgen05 family."""
    from fa_b200 import interface

    for name in DENSE_CASES:
        g = load(name)
        kw = dense_kwargs(g)
        pad = lambda t: torch.nn.functional.pad(t.to(torch.float16), (0, 32)).cuda()
        q, k, v, dout = (pad(g[n]) for n in ("q", "k", "v", "dout"))
        bias = None if kw["bias"] is None else kw["bias"].cuda()
        alibi = None if kw["alibi_slopes"] is None else kw["alibi_slopes"].cuda()
        args = (kw["causal"], kw["softmax_scale"], kw["window"], kw["softcap"], bias, alibi, kw["dropout_p"],
                kw["dropout_seed"])
        with interface.force_kernel_path("tcgen05"):
            out, lse = interface._forward(q, k, v, *args)
            dq, dk, dv = interface._backward(dout, q, k, v, out, lse, *args)
        assert max_abs(out[..., :32], g["out"]) <= 3e-3, name
        assert max_abs(lse, g["lse"]) <= 3e-3, name
        for got, want in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            assert rel_l2(got[..., :32], g[want]) <= 1e-2, (name, want)


def test_decode_golden():
    import fa_b200

    g = load("decode_splitk")
    out = fa_b200.flash_attention_decode(*(g[n].to(torch.float16).cuda() for n in ("q", "k", "v")))
    assert max_abs(out, g["out"]) <= 3e-3


def test_paged_golden():
    import fa_b200

    g = load("decode_paged")
    args = [g[n].to(torch.float16).cuda() for n in ("q", "k_cache", "v_cache")]
    args += [g["block_table"].cuda(), g["context_lens"].cuda()]
    for splits in (1, 3):
        out = fa_b200.flash_attention_decode_paged(*args, num_splits=splits)
        assert max_abs(out, g[f"out_split{splits}"]) <= 3e-3
        assert torch.all(out[2] == 0)


def test_varlen_golden():
    import fa_b200

    g = load("varlen_mods")
    q, k, v = (g[n].to(torch.float16).cuda().requires_grad_(True) for n in ("q", "k", "v"))
    cu = g["cu_seqlens"].cuda()
    lengths = (g["cu_seqlens"][1:] - g["cu_seqlens"][:-1]).tolist()
    out = fa_b200.flash_attention_varlen(q, k, v, cu, cu, max(lengths), max(lengths), causal=True,
                                         window_size=tuple(int(x) for x in g["window"]), softcap=float(g["softcap"]),
                                         alibi_slopes=g["alibi"].cuda())
    out.backward(g["dout"].to(torch.float16).cuda())
    assert max_abs(out, g["out"]) <= 3e-3
    assert rel_l2(q.grad, g["dq"]) <= 1e-2 and rel_l2(k.grad, g["dk"]) <= 1e-2 and rel_l2(v.grad, g["dv"]) <= 1e-2
