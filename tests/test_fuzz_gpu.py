"""Seeded random shapes through the tensor-core kernels, forward and backward, against the fp32 oracle.

The fixed grids of the other files follow the reference's tests; this file walks the corners between them
(ragged lengths around the 128-row tile, cross-attention offsets, windows that start inside a tile, GQA ratios,
empty and one-token sequences in a packed batch, head dims beside 64 and 128 and fp32 inputs, decode and paged-decode
shapes over both kernel families): 48 dense, 64 other-head-dim, 16 packed, 32 decode and 32 paged cases, every one
reproducible from its index.
"""
import random

import pytest
import torch

from test_backward_gpu import run_case
from test_varlen_gpu import run_varlen

pytestmark = pytest.mark.gpu


def dense_case(index):
    rng = random.Random(7000 + index)
    head_dim = rng.choice([64, 128])
    kv_heads = rng.choice([1, 2, 4])
    group = rng.choice([1, 2, 4])
    # lengths cluster around tile edges: 1, 127..129, 255..257, and anything up to 700
    pick = lambda: rng.choice([1, rng.randint(2, 126), 127, 128, 129, rng.randint(130, 254), 255, 256, 257,
                               rng.randint(258, 700)])
    seqlen_q, seqlen_k = pick(), pick()
    opts = {}
    mode = rng.choice(["none", "causal", "window", "causal_window"])
    if mode in ("causal", "causal_window"):
        opts["causal"] = True
    if mode == "window":
        opts["window"] = (rng.randint(0, 300), rng.randint(0, 300))
    if mode == "causal_window":
        opts["window"] = (rng.randint(0, 300), 0)
    dtype = rng.choice([torch.float16, torch.bfloat16])
    return dict(dtype=dtype, B=rng.randint(1, 3), H=kv_heads * group, Hk=kv_heads, Sq=seqlen_q, Sk=seqlen_k,
                D=head_dim, seed=index, **opts)


@pytest.mark.parametrize("index", range(48))
def test_dense_random_shape(index):
    case = dense_case(index)
    used = run_case(path="tcgen05", **case)
    assert used == "tcgen05", case


def other_head_dim_case(index):
    """Head dims beside 64 and 128: narrow and wide 16-bit widths on the tensor-core kernels (zero-filled by the tensor
    maps; above 128 the backward, and above 256 the forward too, are products over tiles in a scratch buffer - above 256
    only without score modifiers), fp32 and the rest on the tiled CUDA-core kernels; lengths around the 64- and 128-row tiles, with modifiers."""
    rng = random.Random(13000 + index)
    kind = ("narrow", "wide", "fp32", "d512")[index % 4]
    dtype = rng.choice([torch.float16, torch.bfloat16])
    if kind == "narrow":
        head_dim = rng.choice([8, 16, 24, 32, 40, 48, 56, 72, 80, 88, 96, 104, 112, 120])
    elif kind == "wide":
        head_dim = rng.choice([136, 144, 160, 176, 192, 200, 224, 248, 256])
    elif kind == "fp32":
        head_dim, dtype = rng.choice([16, 20, 32, 64, 100, 128, 256]), torch.float32
    else:
        head_dim = rng.choice([264, 320, 512])
    kv_heads = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 4])
    seqlen_q = rng.choice([1, 7, 31, 32, 33, 64, 100, 128, 129, 200, 257, 400])
    seqlen_k = rng.choice([1, 5, 63, 64, 65, 128, 130, 255, 256, 300, 513])
    opts = {}
    if rng.random() < 0.5:
        opts["causal"] = True
    if rng.random() < 0.3:
        opts["window"] = (rng.choice([0, 10, 100]), 0 if opts.get("causal") else rng.choice([-1, 0, 20]))
    if rng.random() < 0.3:
        opts["softcap"] = 25.0
    if rng.random() < 0.25:
        opts["alibi"] = True
    # Dropout only where the comparison is well posed: with one visible key per row the exact dQ and dK are zero and
    # what is left is the rounding of O inside delta, and bfloat16 rounds the rescaled probabilities (1 / keep) to 8
    # bits, which alone passes 1e-2 on rows that see a handful of keys.
    if rng.random() < 0.3 and dtype != torch.bfloat16 and seqlen_k >= 63 and "window" not in opts:
        opts["dropout_p"], opts["dropout_seed"] = 0.15, rng.randrange(1 << 20)
    return kind, dict(dtype=dtype, B=rng.randint(1, 2), H=kv_heads * group, Hk=kv_heads, Sq=seqlen_q, Sk=seqlen_k,
                      D=head_dim, seed=index, **opts)


@pytest.mark.parametrize("index", range(64))
def test_other_head_dims_random_shape(index):
    kind, case = other_head_dim_case(index)
    used = run_case(path="auto", **case)   # the path of the backward launch
    plain = not any(name in case for name in ("softcap", "alibi", "dropout_p"))
    assert used == ("tcgen05" if kind in ("narrow", "wide") or (kind == "d512" and plain) else "simt"), case


def packed_case(index):
    rng = random.Random(9000 + index)
    n = rng.randint(2, 6)
    lengths = [rng.choice([0, 1, rng.randint(2, 127), 128, 129, rng.randint(130, 600)]) for _ in range(n)]
    if sum(lengths) == 0:
        lengths[0] = 5
    kv_heads = rng.choice([1, 2])
    group = rng.choice([1, 4])
    opts = rng.choice([dict(), dict(causal=True), dict(causal=True, window=(rng.randint(0, 200), 0))])
    return lengths, kv_heads * group, kv_heads, rng.choice([64, 128]), rng.choice([torch.float16, torch.bfloat16]), opts


@pytest.mark.parametrize("index", range(16))
def test_packed_random_lengths(index):
    lengths, heads, kv_heads, head_dim, dtype, opts = packed_case(index)
    run_varlen(lengths, heads, kv_heads, head_dim, dtype=dtype, path="tcgen05", seed=index, **opts)


# ------------------------------------------------------------------------------------------ decode
def decode_case(index):
    rng = random.Random(11000 + index)
    kv_heads = rng.choice([1, 2, 8])
    group = rng.choice([1, 4])
    seqlen_k = rng.choice([1, 2, 127, 128, 129, 255, 257, rng.randint(300, 3000), 4096, rng.randint(4097, 9000)])
    return dict(batch=rng.randint(1, 3), heads=kv_heads * group, kv_heads=kv_heads, seqlen_q=rng.choice([1, 1, 2, 4]),
                seqlen_k=seqlen_k, head_dim=rng.choice([64, 128]), dtype=rng.choice([torch.float16, torch.bfloat16]),
                splits=rng.choice([1, 2, 3, 4, 8, 16]), path=rng.choice([0, 1, 2]))


@pytest.mark.parametrize("index", range(32))
def test_decode_random_shape(index):
    from fa_b200 import interface
    from helpers import assert_close_o, seeded
    from oracle import attention_oracle as oracle

    c = decode_case(index)
    q = seeded(index + 1, c["batch"], c["heads"], c["seqlen_q"], c["head_dim"], dtype=c["dtype"])
    k = seeded(index + 2, c["batch"], c["kv_heads"], c["seqlen_k"], c["head_dim"], dtype=c["dtype"])
    v = seeded(index + 3, c["batch"], c["kv_heads"], c["seqlen_k"], c["head_dim"], dtype=c["dtype"])
    path = c["path"]
    tc_ok = interface._tensor_core_decode_ok(q, c["head_dim"], c["heads"] // c["kv_heads"] * c["seqlen_q"], 0.1)
    if path == 1 and not (tc_ok and c["splits"] >= 2 and c["splits"] % 2 == 0):
        path = 0  # the tensor-core kernel does not take this case (it wants an even split count): library's choice
    out = interface._decode_impl(q, k, v, 0.1, c["splits"], force_path=path)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.1)
    assert_close_o(out, ref, c["dtype"], str(c))


def paged_case(index):
    rng = random.Random(13000 + index)
    kv_heads = rng.choice([1, 2, 8])
    group = rng.choice([1, 4])
    block_size = rng.choice([8, 16, 32, 64, 128])
    batch = rng.randint(1, 4)
    contexts = [rng.choice([0, 1, block_size - 1, block_size, block_size + 1, rng.randint(2, 3000)]) for _ in range(batch)]
    if max(contexts) == 0:
        contexts[0] = 7
    return dict(batch=batch, heads=kv_heads * group, kv_heads=kv_heads, head_dim=rng.choice([64, 128]),
                block_size=block_size, contexts=contexts, dtype=rng.choice([torch.float16, torch.bfloat16]),
                splits=rng.choice([1, 2, 4, 6, 16]), path=rng.choice([0, 1, 2]))


@pytest.mark.parametrize("index", range(32))
def test_paged_random_shape(index):
    import math

    from fa_b200 import interface
    from helpers import assert_close_o
    from oracle import attention_oracle as oracle
    from test_decode_gpu import make_paged

    c = paged_case(index)
    q, kc, vc, table, ctx = make_paged(c["batch"], c["heads"], c["kv_heads"], c["head_dim"], c["block_size"],
                                       c["contexts"], dtype=c["dtype"], seed=index)
    scale = 1.0 / math.sqrt(c["head_dim"])
    path = c["path"]
    tc_ok = interface._paged_tensor_core_ok(q, c["head_dim"], c["heads"], c["kv_heads"], c["block_size"], scale)
    if path == 1 and not (tc_ok and c["splits"] >= 2 and c["splits"] % 2 == 0):
        path = 0
    out, _ = interface._paged_launch(q, kc, vc, table, ctx, scale, c["splits"], force_path=path)
    ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu())
    assert_close_o(out, ref, c["dtype"], str(c))
