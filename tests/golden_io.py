"""Loader for tests/golden/*.npz (outputs of the reference's own kernels; see tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DENSE_CASES = ["dense_causal_cross", "dense_gqa_causal", "dense_mods", "dense_empty_rows", "dense_dropout"]


def load(name):
    data = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(data[k])) if data[k].ndim else data[k].item() for k in data.files}


def dense_kwargs(g):
    """Keyword arguments of oracle.attention_ref for a dense golden case."""
    window = tuple(int(x) for x in g["window"])
    return dict(causal=bool(g["causal"]), softmax_scale=float(g["scale"]), window=window,
                softcap=float(g["softcap"]), bias=g.get("bias"), alibi_slopes=g.get("alibi"),
                dropout_p=float(g["dropout_p"]), dropout_seed=int(g["dropout_seed"]))
