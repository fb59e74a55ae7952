"""Pins the CPU oracle to outputs of the reference's own kernels (tests/golden/*.npz).

The goldens are fp16 results of the reference's Triton kernels run under the Triton interpreter, so the
comparison uses fp16-level tolerances: 3e-3 absolute on O / LSE (the reference's own bound,
tests/test_forward.py:29-30) and 1e-2 relative L2 on gradients.
"""
import pytest
import torch

from golden_io import DENSE_CASES, dense_kwargs, load
from helpers import max_abs, rel_l2
from oracle import attention_oracle as oracle


@pytest.mark.parametrize("name", DENSE_CASES)
def test_dense_forward_backward_matches_reference(name):
    g = load(name)
    half = lambda t: t.to(torch.float16)
    out, lse, dq, dk, dv = oracle.attention_grads_ref(half(g["q"]), half(g["k"]), half(g["v"]), half(g["dout"]),
                                                      **dense_kwargs(g))
    assert max_abs(out, g["out"]) <= 3e-3
    assert max_abs(lse, g["lse"]) <= 3e-3
    assert rel_l2(dq, g["dq"]) <= 1e-2
    assert rel_l2(dk, g["dk"]) <= 1e-2
    assert rel_l2(dv, g["dv"]) <= 1e-2


def test_empty_rows_are_zero_with_neg_inf_lse():
    g = load("dense_empty_rows")
    # Sq = 72 > Sk = 40 with a bottom-right causal mask: the first 32 rows see no key
    assert torch.all(g["out"][:, :, :32] == 0)
    assert torch.all(torch.isinf(g["lse"][:, :, :32]) & (g["lse"][:, :, :32] < 0))
    out, lse = oracle.attention_ref(g["q"], g["k"], g["v"], **dense_kwargs(g))
    assert torch.all(out[:, :, :32] == 0) and torch.all(torch.isinf(lse[:, :, :32]))


def test_dropout_mask_bits_match_reference():
    # With the wrong mask the outputs differ by O(1); agreement at 3e-3 pins the Philox stream.
    g = load("dense_dropout")
    kw = dense_kwargs(g)
    out, _ = oracle.attention_ref(g["q"], g["k"], g["v"], **kw)
    assert max_abs(out, g["out"]) <= 3e-3
    kw["dropout_seed"] += 1
    other, _ = oracle.attention_ref(g["q"], g["k"], g["v"], **kw)
    assert max_abs(other, g["out"]) > 5e-2


def test_decode_matches_reference():
    g = load("decode_splitk")
    out, _ = oracle.decode_ref(g["q"], g["k"], g["v"])
    assert max_abs(out, g["out"]) <= 3e-3


def test_paged_matches_reference():
    g = load("decode_paged")
    out, _ = oracle.paged_ref(g["q"], g["k_cache"], g["v_cache"], g["block_table"], g["context_lens"])
    assert max_abs(out, g["out_split1"]) <= 3e-3
    assert max_abs(out, g["out_split3"]) <= 3e-3
    assert torch.all(g["out_split3"][2] == 0)  # context_len 0 -> zeros


def test_paged_shards_merge_to_whole():
    g = load("decode_paged")
    parts = [oracle.paged_ref(g["q"], g["k_cache"], g["v_cache"], g["block_table"], g["context_lens"],
                              first_block=r, block_step=3) for r in range(3)]
    o, _ = oracle.combine_ref(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert max_abs(o, g["out_split1"]) <= 3e-3


def test_varlen_matches_reference():
    g = load("varlen_mods")
    half = lambda t: t.to(torch.float16)
    cu = g["cu_seqlens"]
    out, lse, dq, dk, dv = oracle.varlen_grads_ref(
        half(g["q"]), half(g["k"]), half(g["v"]), half(g["dout"]), cu, cu, causal=True,
        window=tuple(int(x) for x in g["window"]), softcap=float(g["softcap"]), alibi_slopes=g["alibi"])
    assert max_abs(out, g["out"]) <= 3e-3
    assert rel_l2(dq, g["dq"]) <= 1e-2
    assert rel_l2(dk, g["dk"]) <= 1e-2
    assert rel_l2(dv, g["dv"]) <= 1e-2


def test_combine_closed_form():
    # two partials with equal LSE average; a -inf partial is ignored; all -inf gives zeros
    o = torch.tensor([[[1.0, 3.0]], [[3.0, 5.0]], [[100.0, 100.0]]])
    lse = torch.tensor([[0.5], [0.5], [float("-inf")]])
    out, l = oracle.combine_ref(o, lse)
    assert torch.allclose(out, torch.tensor([[2.0, 4.0]]))
    assert torch.allclose(l, torch.tensor([0.5 + 0.6931472]))
    out, l = oracle.combine_ref(o, torch.full((3, 1), float("-inf")))
    assert torch.all(out == 0) and torch.isinf(l).all()


def test_alibi_slopes_closed_form():
    s = oracle.alibi_slopes_ref(32)
    want = torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)])
    assert torch.allclose(s, want, rtol=1e-6)
    assert oracle.alibi_slopes_ref(12).shape == (12,)
