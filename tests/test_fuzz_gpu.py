"""Seeded random shapes through the tensor-core kernels, forward and backward, against the fp32 oracle.

The fixed grids of the other files follow the reference's tests; this file walks the corners between them
(ragged lengths around the 128-row tile, cross-attention offsets, windows that start inside a tile, GQA ratios,
empty and one-token sequences in a packed batch), 48 dense and 16 packed cases, every one reproducible from its index.
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
