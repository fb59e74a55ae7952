"""Generate tests/golden/*.npz from the reference package itself.

Run where a checkout of the reference (chelokot/flash-attention-rdna3) and Triton are available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py <path to the reference checkout>

The reference's Triton kernels are executed on CPU tensors by Triton's interpreter, through the
reference's own public functions and launch glue. Three things are patched, none of which touches the
arithmetic: the ROCm/gfx1100 platform gate is disabled (the reference's own CPU tests do the same), the
autotuner is bypassed by launching each kernel's undecorated function with one fixed tile shape (the
reference's sweep scripts launch kernels this way), and the SM-count query is answered with 148.
The FP32 short-sequence kernel does not run under the interpreter and has no golden file.

Each .npz holds the seeded inputs and the reference's outputs, so the fixtures are self-contained.
"""
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path to the reference checkout>")
REF = sys.argv[1]
sys.path.insert(0, REF)

import numpy as np
import torch

import fa_rdna3
from fa_rdna3 import _validation, interface, kernels

OUT = os.path.dirname(os.path.abspath(__file__))

_validation._require_platform = lambda device: None
torch.cuda.get_device_properties = lambda device=None: types.SimpleNamespace(multi_processor_count=148)


class FixedTile:
    """Stands in for an autotuned kernel: launches its plain jit function with fixed meta-parameters."""

    def __init__(self, autotuned, **meta):
        self.fn = autotuned.fn
        self.meta = meta

    def __getitem__(self, grid):
        g = grid(self.meta) if callable(grid) else grid

        def launch(*args, **kw):
            return self.fn[g](*args, **{**kw, **self.meta})

        return launch


interface._attention_forward = FixedTile(kernels._attention_forward, BLOCK_M=32, BLOCK_N=32)
interface._attention_bwd_dkdv = FixedTile(kernels._attention_bwd_dkdv, BLOCK_M=32, BLOCK_N=32)
interface._attention_bwd_dq = FixedTile(kernels._attention_bwd_dq, BLOCK_M=32, BLOCK_N=32)
interface._attention_split = FixedTile(kernels._attention_split, BLOCK_N=32)
interface._attention_forward_varlen = FixedTile(kernels._attention_forward_varlen, BLOCK_M=32, BLOCK_N=32)
interface._attention_bwd_dkdv_varlen = FixedTile(kernels._attention_bwd_dkdv_varlen, BLOCK_M=32, BLOCK_N=32)
interface._attention_bwd_dq_varlen = FixedTile(kernels._attention_bwd_dq_varlen, BLOCK_M=32, BLOCK_N=32)


def randn(gen, *shape, dtype=torch.float16):
    return torch.randn(*shape, generator=gen, dtype=torch.float32).to(dtype)


def save(name, **arrays):
    conv = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach()
            v = v.float().numpy() if v.dtype in (torch.float16, torch.bfloat16) else v.numpy()
        conv[k] = np.asarray(v)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **conv)
    print("wrote", name, {k: tuple(np.shape(v)) for k, v in conv.items()})


def dense_fwd_bwd(name, seed, B, H, Hk, Sq, Sk, D, **opts):
    g = torch.Generator().manual_seed(seed)
    q, k, v = randn(g, B, H, Sq, D), randn(g, B, Hk, Sk, D), randn(g, B, Hk, Sk, D)
    dout = randn(g, B, H, Sq, D)
    scale = 1.0 / D ** 0.5
    window = opts.get("window", (-1, -1))
    softcap = opts.get("softcap", 0.0)
    bias = opts.get("bias")
    if bias == "random":
        bias = torch.randn(1, H, Sq, Sk, generator=g)
        bias[..., : Sk // 3] = float("-inf") if opts.get("mask_prefix") else bias[..., : Sk // 3]
    alibi = fa_rdna3.alibi_slopes(H, device="cpu") if opts.get("alibi") else None
    p, dseed = opts.get("dropout_p", 0.0), opts.get("dropout_seed", 0)
    causal = opts.get("causal", False)
    out, lse = interface._forward(q, k, v, causal, scale, window, softcap, bias, alibi, p, dseed)
    dq, dk, dv = interface._backward(dout, q, k, v, out, lse, causal, scale, window, softcap, bias, alibi, p, dseed)
    extra = {}
    if bias is not None:
        extra["bias"] = bias
    if alibi is not None:
        extra["alibi"] = alibi
    save(name, q=q, k=k, v=v, dout=dout, out=out, lse=lse, dq=dq, dk=dk, dv=dv, scale=scale, causal=int(causal),
         window=np.array(window), softcap=softcap, dropout_p=p, dropout_seed=dseed, **extra)


def main():
    dense_fwd_bwd("dense_causal_cross", 11, 1, 2, 2, 48, 80, 32, causal=True)
    dense_fwd_bwd("dense_gqa_causal", 12, 1, 4, 2, 64, 64, 32, causal=True)
    dense_fwd_bwd("dense_mods", 13, 1, 4, 2, 40, 72, 32, window=(9, 5), softcap=30.0, alibi=True, bias="random")
    dense_fwd_bwd("dense_empty_rows", 14, 1, 2, 2, 72, 40, 32, causal=True)  # Sq > Sk: rows without keys
    dense_fwd_bwd("dense_dropout", 15, 2, 2, 2, 40, 56, 32, dropout_p=0.25, dropout_seed=1234)

    # split-K decode
    g = torch.Generator().manual_seed(21)
    q, k, v = randn(g, 2, 4, 2, 64), randn(g, 2, 2, 300, 64), randn(g, 2, 2, 300, 64)
    out = fa_rdna3.flash_attention_decode(q, k, v)
    save("decode_splitk", q=q, k=k, v=v, out=out)

    # paged decode, GQA, shuffled pages, several splits
    g = torch.Generator().manual_seed(22)
    B, Hq, Hk, D, bs, maxb = 3, 4, 2, 32, 8, 6
    nblocks = B * maxb
    q = randn(g, B, Hq, D)
    kc, vc = randn(g, nblocks, bs, Hk, D), randn(g, nblocks, bs, Hk, D)
    table = torch.randperm(nblocks, generator=g).to(torch.int32).reshape(B, maxb)
    ctx = torch.tensor([41, 8, 0], dtype=torch.int32)
    out1 = fa_rdna3.flash_attention_decode_paged(q, kc, vc, table, ctx, num_splits=1)
    out3 = fa_rdna3.flash_attention_decode_paged(q, kc, vc, table, ctx, num_splits=3)
    save("decode_paged", q=q, k_cache=kc, v_cache=vc, block_table=table, context_lens=ctx, out_split1=out1,
         out_split3=out3)

    # packed varlen with window + softcap + ALiBi, forward and backward
    g = torch.Generator().manual_seed(23)
    lengths = [37, 5, 64, 1]
    total = sum(lengths)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    Hq, Hk, D = 4, 2, 32
    q = randn(g, total, Hq, D).requires_grad_(True)
    k = randn(g, total, Hk, D).requires_grad_(True)
    v = randn(g, total, Hk, D).requires_grad_(True)
    dout = randn(g, total, Hq, D)
    slopes = fa_rdna3.alibi_slopes(Hq, device="cpu")
    out = fa_rdna3.flash_attention_varlen(q, k, v, cu, cu, max(lengths), max(lengths), causal=True,
                                          window_size=(15, 0), softcap=30.0, alibi_slopes=slopes)
    out.backward(dout)
    save("varlen_mods", q=q, k=k, v=v, dout=dout, cu_seqlens=cu, out=out, dq=q.grad, dk=k.grad, dv=v.grad,
         alibi=slopes, window=np.array([15, 0]), softcap=30.0)


if __name__ == "__main__":
    main()
