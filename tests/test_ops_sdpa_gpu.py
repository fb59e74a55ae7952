"""torch.library registration (opcheck, torch.compile) and the scaled_dot_product_attention hook on the GPU.
Modelled on the reference's tests/test_torch_library.py, tests/test_tiny.py:67-92 and tests/test_sdpa_dispatch.py."""
import math

import pytest
import torch
import torch.nn.functional as F

from helpers import max_abs, seeded

pytestmark = pytest.mark.gpu


def test_opcheck_flash_fwd():
    import fa_b200  # noqa: F401

    q, k, v = (seeded(i, 1, 2, 128, 64).requires_grad_(True) for i in (1, 2, 3))
    args = (q, k, v, True, 0.125, -1, -1, 0.0, None, None, 0.0, 0)
    torch.library.opcheck(torch.ops.fa_b200.flash_fwd.default, args,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_opcheck_tiny_and_decode_ops():
    import fa_b200  # noqa: F401

    q = seeded(1, 1, 2, 6, 128, dtype=torch.float32)
    torch.library.opcheck(torch.ops.fa_b200.flash_tiny_fwd.default, (q, q, q, 0.0884, None, 8),
                          test_utils=("test_schema", "test_faketensor"))
    qd, kd = seeded(2, 1, 4, 1, 64), seeded(3, 1, 2, 512, 64)
    torch.library.opcheck(torch.ops.fa_b200.decode_splitk.default, (qd, kd, kd, 0.125, 2),
                          test_utils=("test_schema", "test_faketensor"))


def test_compile_matches_eager_forward_and_backward():
    import fa_b200

    def f(q, k, v):
        return fa_b200.flash_attention(q, k, v, causal=True)

    q, k, v = (seeded(i, 1, 4, 256, 64).requires_grad_(True) for i in (1, 2, 3))
    eager = f(q, k, v)
    g_eager = torch.autograd.grad(eager.float().sum(), (q, k, v))
    compiled = torch.compile(f, fullgraph=True)(q, k, v)
    g_comp = torch.autograd.grad(compiled.float().sum(), (q, k, v))
    assert torch.equal(eager, compiled)
    assert all(torch.equal(a, b) for a, b in zip(g_eager, g_comp))


def test_tiny_fp32_under_compile_matches_stock_sdpa():
    import fa_b200

    q, k, v = (seeded(i, 2, 8, 19, 128, dtype=torch.float32) for i in (1, 2, 3))
    want = F.scaled_dot_product_attention(q, k, v)

    def f(q, k, v):
        return F.scaled_dot_product_attention(q, k, v)

    with fa_b200.use_flash_attention():
        got = torch.compile(f, fullgraph=True)(q, k, v)
    assert max_abs(got, want) <= 5e-6


@pytest.mark.parametrize("is_causal", [False, True])
def test_sdpa_hook_matches_stock(is_causal):
    import fa_b200
    from fa_b200 import interface

    q, k, v = (seeded(i, 2, 8, 512, 64) for i in (1, 2, 3))
    want = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=is_causal)
    with fa_b200.use_flash_attention():
        got = F.scaled_dot_product_attention(q, k, v, is_causal=is_causal)
    assert interface.last_kernel_path() == "tcgen05"
    assert max_abs(got, want) <= 2e-3


def test_sdpa_hook_bool_mask_gqa_and_decode_route(monkeypatch):
    import fa_b200
    from fa_b200 import sdpa

    q, k, v = seeded(1, 1, 8, 100, 64), seeded(2, 1, 2, 130, 64), seeded(3, 1, 2, 130, 64)
    mask = torch.rand(1, 1, 100, 130, device="cuda") > 0.3
    mask[..., 0] = True
    want = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask, enable_gqa=True)
    with fa_b200.use_flash_attention():
        got = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=True)
    assert max_abs(got, want) <= 2e-3

    calls = []
    real = sdpa.flash_attention_decode
    monkeypatch.setattr(sdpa, "flash_attention_decode", lambda *a, **kw: calls.append(1) or real(*a, **kw))
    qd, kd, vd = seeded(4, 2, 8, 1, 128), seeded(5, 2, 8, 2048, 128), seeded(6, 2, 8, 2048, 128)
    want = F.scaled_dot_product_attention(qd.float(), kd.float(), vd.float())
    with fa_b200.use_flash_attention():
        got = F.scaled_dot_product_attention(qd, kd, vd)
    assert calls == [1] and max_abs(got, want) <= 2e-3


def test_sdpa_hook_falls_back_for_unsupported_calls():
    import fa_b200

    q = seeded(1, 1, 2, 64, 64, dtype=torch.float32).double()
    with fa_b200.use_flash_attention():
        out = F.scaled_dot_product_attention(q, q, q)          # float64: original implementation
        out2 = F.scaled_dot_product_attention(q.half(), q.half(), q.half(), dropout_p=0.5)  # dropout: original
    assert out.dtype == torch.float64 and out2.shape == q.shape
