"""Packed variable-length attention forward and backward against the per-sequence oracle.

Modelled on the reference's tests/test_varlen.py and tests/test_varlen_mods.py.
"""
import pytest
import torch

from helpers import assert_close_grad, assert_close_o, max_abs, seeded
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu


def cu_of(lengths):
    return torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)


def run_varlen(lengths, Hq, Hk, D, dtype=torch.float16, path="auto", seed=0, **opts):
    import fa_b200
    from fa_b200 import interface

    total = sum(lengths)
    q = seeded(seed + 1, total, Hq, D, dtype=dtype).requires_grad_(True)
    k = seeded(seed + 2, total, Hk, D, dtype=dtype).requires_grad_(True)
    v = seeded(seed + 3, total, Hk, D, dtype=dtype).requires_grad_(True)
    dout = seeded(seed + 4, total, Hq, D, dtype=dtype)
    cu = cu_of(lengths)
    slopes = oracle.alibi_slopes_ref(Hq) if opts.get("alibi") else None
    kw = dict(causal=opts.get("causal", False), window_size=opts.get("window", (-1, -1)),
              softcap=opts.get("softcap", 0.0))
    with interface.force_kernel_path(path):
        out = fa_b200.flash_attention_varlen(q, k, v, cu.cuda(), cu.cuda(), max(lengths), max(lengths),
                                             alibi_slopes=None if slopes is None else slopes.cuda(), **kw)
        out.backward(dout)
    torch.cuda.synchronize()
    ro, _, rdq, rdk, rdv = oracle.varlen_grads_ref(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), dout.cpu(),
                                                   cu, cu, causal=kw["causal"], window=kw["window_size"],
                                                   softcap=kw["softcap"], alibi_slopes=slopes)
    assert_close_o(out, ro, dtype)
    assert_close_grad(q.grad, rdq, "dq")
    assert_close_grad(k.grad, rdk, "dk")
    assert_close_grad(v.grad, rdv, "dv")


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_basic(path, causal):
    run_varlen([128, 57, 300, 1], 4, 4, 64, path=path, causal=causal)


@pytest.mark.parametrize("path", ["tcgen05", "simt"])
@pytest.mark.parametrize("opts", [dict(causal=True, window=(31, 0)), dict(softcap=30.0),
                                  dict(causal=True, alibi=True),
                                  dict(causal=True, window=(255, 0), softcap=30.0, alibi=True)])
def test_varlen_modifiers(path, opts):
    run_varlen([200, 64, 333, 7], 8, 2, 128, path=path, seed=3, **opts)


def test_varlen_long_bf16_gqa():
    run_varlen([1500, 700, 2048, 129], 8, 2, 128, dtype=torch.bfloat16, seed=5, causal=True)


def test_varlen_equals_padded_batched():
    import fa_b200

    L, B, H, D = 256, 3, 4, 64
    q, k, v = (seeded(i, B * L, H, D) for i in (1, 2, 3))
    cu = cu_of([L] * B).cuda()
    packed = fa_b200.flash_attention_varlen(q, k, v, cu, cu, L, L, causal=True)
    dense = fa_b200.flash_attention(*(t.view(B, L, H, D).transpose(1, 2) for t in (q, k, v)), causal=True)
    assert max_abs(packed.view(B, L, H, D).transpose(1, 2), dense) <= 1e-3


def test_varlen_cross_attention_lengths():
    import fa_b200

    lq, lk = [50, 200, 3], [300, 64, 129]
    q = seeded(1, sum(lq), 4, 64)
    k, v = seeded(2, sum(lk), 2, 64), seeded(3, sum(lk), 2, 64)
    out = fa_b200.flash_attention_varlen(q, k, v, cu_of(lq).cuda(), cu_of(lk).cuda(), max(lq), max(lk), causal=True)
    ref, _ = oracle.varlen_ref(q.cpu(), k.cpu(), v.cpu(), cu_of(lq), cu_of(lk), causal=True)
    assert_close_o(out, ref, torch.float16)


def test_varlen_out_of_range_metadata_is_clamped():
    import fa_b200

    q, k, v = (seeded(i, 300, 4, 64) for i in (1, 2, 3))
    cu = torch.tensor([-7, 100, 250, 900], dtype=torch.int32)  # clamped to [0, 300]
    out = fa_b200.flash_attention_varlen(q, k, v, cu.cuda(), cu.cuda(), 300, 300, causal=True)
    ref, _ = oracle.varlen_ref(q.cpu(), k.cpu(), v.cpu(), cu, cu, causal=True)
    assert_close_o(out, ref, torch.float16)


@pytest.mark.parametrize("count", [40, 128, 140])
def test_varlen_many_sequences_with_empty_ones(count):
    """Packed batches on the compact grid: CTAs find their (sequence, tile) from cu_seqlens, 32 sequences per ballot.
    40 sequences take two ballots, 128 is the most the compact grid takes, 140 falls back to one CTA per (sequence,
    possible tile); every third sequence is empty, one is much longer than the rest."""
    import random

    rng = random.Random(count)
    lengths = [0 if i % 3 == 1 else rng.randint(1, 70) for i in range(count)]
    lengths[count // 2] = 700
    run_varlen(lengths, 4, 2, 64, path="tcgen05", causal=True, seed=count)
