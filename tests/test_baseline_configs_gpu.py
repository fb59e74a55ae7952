"""The five benchmark configurations at their full sizes, with the seeds and shapes stated for them.

The oracle (fp32 math attention) is evaluated on the GPU here so the full sizes finish in seconds; matmuls stay in
true fp32 (TF32 is switched off explicitly). Small-size cases elsewhere run the same oracle on the CPU.
Tolerances: O / LSE max-abs 2e-3 (fp16) or 1e-2 (bf16); gradients relative L2 1e-2.
"""
import math

import pytest
import torch

from helpers import assert_close_grad, assert_close_o, excess_over_tolerance, max_abs, rel_l2
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _true_fp32():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old


def gen(seed):
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, dtype=torch.float16):
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype).cuda()


def test_c1_forward_noncausal_1x16x1024x64():
    from fa_b200 import interface

    g = gen(1001)
    q, k, v = (randn(g, 1, 16, 1024, 64) for _ in range(3))
    out, lse = interface._forward(q, k, v, False, 1 / 8, (-1, -1), 0.0, None, None, 0.0, 0)
    assert interface.last_kernel_path() == "tcgen05"
    ro, rl = oracle.attention_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=1 / 8)  # CPU oracle at this size
    assert_close_o(out, ro, torch.float16)
    assert_close_o(lse, rl, torch.float16, "lse")


@pytest.mark.parametrize("seed,shape", [(1002, (2, 16, 2048, 128)), (1003, (1, 16, 4096, 64))])
def test_c2_forward_backward_causal(seed, shape):
    from fa_b200 import interface

    g = gen(seed)
    q, k, v, dout = (randn(g, *shape) for _ in range(4))
    scale = 1 / math.sqrt(shape[-1])
    out, lse = interface._forward(q, k, v, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    dq, dk, dv = interface._backward(dout, q, k, v, out, lse, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    assert interface.last_kernel_path() == "tcgen05"
    ro, rl, rdq, rdk, rdv = oracle.attention_grads_ref(q, k, v, dout, causal=True, softmax_scale=scale)
    assert_close_o(out, ro, torch.float16)
    assert_close_o(lse, rl, torch.float16, "lse")
    assert_close_grad(dq, rdq, "dq")
    assert_close_grad(dk, rdk, "dk")
    assert_close_grad(dv, rdv, "dv")


@pytest.mark.parametrize("seed,B,H,Sk", [(1004, 4, 32, 8192), (1005, 1, 8, 16384)])
def test_c3_split_k_decode(seed, B, H, Sk):
    import fa_b200

    g = gen(seed)
    q = randn(g, B, H, 1, 128)
    k, v = randn(g, B, H, Sk, 128), randn(g, B, H, Sk, 128)
    out = fa_b200.flash_attention_decode(q, k, v)
    ref, _ = oracle.decode_ref(q, k, v)
    assert_close_o(out, ref, torch.float16)


def test_c4_paged_decode_gqa_random_pages_and_contexts():
    import fa_b200

    g = gen(1006)
    ctx = torch.randint(1, 16385, (4,), generator=g).to(torch.int32)
    kc, vc = randn(g, 4096, 16, 8, 128), randn(g, 4096, 16, 8, 128)
    table = torch.randperm(4096, generator=g).to(torch.int32).reshape(4, 1024)
    q = randn(g, 4, 32, 128)
    out = fa_b200.flash_attention_decode_paged(q, kc, vc, table.cuda(), ctx.cuda(), max_context_len=16384)
    ref, _ = oracle.paged_ref(q, kc, vc, table, ctx)
    assert_close_o(out, ref, torch.float16)
    # the KV-sharded form (every 2nd / 4th / 8th logical block per shard) merges to the same result
    from fa_b200 import interface

    for G in (2, 8):
        parts = [interface._paged_launch(q, kc, vc, table.cuda(), ctx.cuda(), 1 / math.sqrt(128), 4, first_block=r,
                                         block_step=G, want_lse=True, out_f32=True) for r in range(G)]
        o, _ = oracle.combine_ref(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
        assert max_abs(o, ref) <= 2e-3


def test_c5_varlen_causal_window_alibi_softcap_bf16():
    import fa_b200
    from fa_b200 import interface

    seed = 1007
    while True:
        g = gen(seed)
        lengths = torch.randint(128, 4097, (8,), generator=g).tolist()
        if sum(lengths) <= 16384:
            break
        seed += 1
    T = sum(lengths)
    q = randn(g, T, 32, 128, dtype=torch.bfloat16).requires_grad_(True)
    k = randn(g, T, 8, 128, dtype=torch.bfloat16).requires_grad_(True)
    v = randn(g, T, 8, 128, dtype=torch.bfloat16).requires_grad_(True)
    dout = randn(g, T, 32, 128, dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    slopes = fa_b200.alibi_slopes(32)
    out = fa_b200.flash_attention_varlen(q, k, v, cu.cuda(), cu.cuda(), max(lengths), max(lengths), causal=True,
                                         window_size=(1023, 0), softcap=30.0, alibi_slopes=slopes)
    out.backward(dout)
    assert interface.last_kernel_path() == "tcgen05"
    # oracle one sequence at a time on the GPU (fp32), to bound memory
    worst = {"o": -1.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    for b, L in enumerate(lengths):
        s = int(cu[b])
        sl = slice(s, s + L)
        qb, kb, vb, db = (t.detach()[sl].transpose(0, 1).unsqueeze(0) for t in (q, k, v, dout))
        ro, _, rdq, rdk, rdv = oracle.attention_grads_ref(qb, kb, vb, db, causal=True, window=(1023, 0), softcap=30.0,
                                                          alibi_slopes=slopes)
        ro_abs = oracle.attention_ref(qb, kb, vb.abs(), causal=True, window=(1023, 0), softcap=30.0,
                                      alibi_slopes=slopes)[0]
        worst["o"] = max(worst["o"], excess_over_tolerance(out.detach()[sl].transpose(0, 1), ro[0], torch.bfloat16,
                                                           weighted_abs_v=ro_abs[0]))
        worst["dq"] = max(worst["dq"], rel_l2(q.grad[sl].transpose(0, 1), rdq[0]))
        worst["dk"] = max(worst["dk"], rel_l2(k.grad[sl].transpose(0, 1), rdk[0]))
        worst["dv"] = max(worst["dv"], rel_l2(v.grad[sl].transpose(0, 1), rdv[0]))
    assert worst["o"] <= 0, worst  # 1e-2, or the bfloat16 rounding bound of helpers.excess_over_tolerance
    assert max(worst["dq"], worst["dk"], worst["dv"]) <= 1e-2, worst
