"""Input contracts: exception classes and messages, checked on CPU with the platform gate patched out
(the reference's tests/test_validation.py does the same)."""
import pytest
import torch

import fa_b200
from fa_b200 import _validation, interface


@pytest.fixture
def no_gate(monkeypatch):
    monkeypatch.setattr(_validation, "_require_platform", lambda device: None)


def t(*shape, dtype=torch.float16):
    return torch.zeros(*shape, dtype=dtype)


@pytest.mark.skipif(torch.cuda.is_available(), reason="describes a machine without a GPU")
def test_platform_gate_message_on_cpu():
    assert fa_b200.unsupported_reason() is not None
    assert not fa_b200.is_available()
    with pytest.raises(RuntimeError, match="fa-b200 requires"):
        fa_b200.flash_attention(t(1, 1, 4, 16), t(1, 1, 4, 16), t(1, 1, 4, 16))


def test_gate_accepts_compute_capability_10(monkeypatch):
    monkeypatch.setattr(_validation, "_supported_devices", set())   # the gate remembers devices it has accepted
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(_validation, "_device_arch", lambda index: (10, 0))
    assert fa_b200.unsupported_reason("cuda:0") is None
    monkeypatch.setattr(_validation, "_device_arch", lambda index: (9, 0))
    monkeypatch.setattr(_validation, "_supported_devices", set())
    assert "compute capability 10.x" in fa_b200.unsupported_reason("cuda:0")
    assert "CUDA GPU tensor" in fa_b200.unsupported_reason("cpu")


@pytest.mark.parametrize("args,exc,msg", [
    ((t(1, 4, 16), t(1, 1, 4, 16), t(1, 1, 4, 16)), ValueError, "query must have shape"),
    ((t(1, 1, 4, 16, dtype=torch.float64),) * 3, ValueError, "unsupported dtype"),
    ((t(1, 1, 4, 16), t(1, 1, 4, 16, dtype=torch.bfloat16), t(1, 1, 4, 16)), ValueError, "same dtype"),
    ((t(2, 1, 4, 16), t(1, 1, 4, 16), t(1, 1, 4, 16)), ValueError, "same batch size"),
    ((t(1, 2, 4, 16), t(1, 2, 4, 16), t(1, 1, 4, 16)), ValueError, "same number of heads"),
    ((t(1, 1, 4, 16), t(1, 1, 5, 16), t(1, 1, 4, 16)), ValueError, "same sequence length"),
    ((t(1, 1, 4, 16), t(1, 1, 4, 32), t(1, 1, 4, 32)), ValueError, "same head_dim"),
    ((t(1, 1, 4, 1024),) * 3, ValueError, "exceeds the supported maximum"),
    ((t(1, 3, 4, 16), t(1, 2, 4, 16), t(1, 2, 4, 16)), ValueError, "multiple of key/value heads"),
    (("q", t(1, 1, 4, 16), t(1, 1, 4, 16)), TypeError, "must be a torch.Tensor"),
])
def test_dense_contracts(no_gate, args, exc, msg):
    with pytest.raises(exc, match=msg):
        fa_b200.flash_attention(*args)


@pytest.mark.parametrize("kw,exc,msg", [
    (dict(softmax_scale="1"), TypeError, "softmax_scale must be a real number"),
    (dict(softmax_scale=float("nan")), ValueError, "softmax_scale must be finite"),
    (dict(window_size=(1,)), ValueError, "exactly \\(left, right\\)"),
    (dict(window_size=(-2, 0)), ValueError, "greater than or equal to -1"),
    (dict(window_size=(True, 0)), ValueError, "greater than or equal to -1"),
    (dict(softcap=-1.0), ValueError, "softcap must be nonnegative"),
    (dict(softcap=float("inf")), ValueError, "finite nonnegative"),
    (dict(dropout_p=1.0), ValueError, "0 <= dropout_p < 1"),
    (dict(bias=torch.zeros(3, 3)), ValueError, "broadcastable"),
    (dict(bias=torch.zeros(4, 4, dtype=torch.float64)), ValueError, "bias dtype"),
    (dict(bias=torch.zeros(4, 4, requires_grad=True)), ValueError, "bias gradients"),
    (dict(alibi_slopes=torch.zeros(3)), ValueError, "alibi_slopes must have shape \\(2,\\)"),
    (dict(alibi_slopes=torch.zeros(2, dtype=torch.int32)), ValueError, "floating-point"),
    (dict(alibi_slopes=torch.zeros(2, requires_grad=True)), ValueError, "ALiBi slope gradients"),
])
def test_option_contracts(no_gate, kw, exc, msg):
    q = t(1, 2, 4, 16)
    with pytest.raises(exc, match=msg):
        fa_b200.flash_attention(q, q, q, **kw)


def test_head_dim_padding_limit(no_gate, monkeypatch):
    monkeypatch.setattr(interface, "_SUPPORTED_HEAD_DIMS", (16, 32, 64, 128, 256))
    q = t(1, 1, 4, 300)
    with pytest.raises(ValueError, match="would pad to 512"):
        fa_b200.flash_attention(q, q, q)


def test_decode_contracts(no_gate):
    q = t(1, 2, 1, 48)
    with pytest.raises(ValueError, match="head_dim 48 not supported"):
        fa_b200.flash_attention_decode(q, q, q)
    qg = t(1, 2, 1, 64).requires_grad_(True)
    with pytest.raises(RuntimeError, match="inference-only"):
        fa_b200.flash_attention_decode(qg, qg, qg)
    with pytest.raises(ValueError, match="unsupported dtype"):
        fa_b200.flash_attention_decode(q.float(), q.float(), q.float())


def test_varlen_contracts(no_gate):
    q, k = t(10, 4, 64), t(10, 2, 64)
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    f = fa_b200.flash_attention_varlen
    with pytest.raises(ValueError, match="total_tokens, heads, head_dim"):
        f(t(1, 10, 4, 64), k, k, cu, cu, 6, 6)
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        f(q.float(), k.float(), k.float(), cu, cu, 6, 6)
    with pytest.raises(ValueError, match="same shape"):
        f(q, k, t(9, 2, 64), cu, cu, 6, 6)
    with pytest.raises(ValueError, match="multiple of key/value heads"):
        f(q, t(10, 3, 64), t(10, 3, 64), cu, cu, 6, 6)
    with pytest.raises(ValueError, match="is not supported by varlen"):
        f(t(10, 4, 48), t(10, 2, 48), t(10, 2, 48), cu, cu, 6, 6)
    with pytest.raises(ValueError, match="contiguous int32"):
        f(q, k, k, cu.long(), cu, 6, 6)
    with pytest.raises(ValueError, match="shape \\(batch \\+ 1,\\)"):
        f(q, k, k, cu[:1], cu[:1], 6, 6)
    with pytest.raises(ValueError, match="same batch size"):
        f(q, k, k, cu, cu[:2], 6, 6)
    with pytest.raises(ValueError, match="max_seqlen_q must be a positive integer"):
        f(q, k, k, cu, cu, 0, 6)
    with pytest.raises(ValueError, match="max_seqlen_k must be a positive integer"):
        f(q, k, k, cu, cu, 6, 11)


def test_paged_contracts(no_gate):
    q, kc = t(2, 4, 64), t(8, 16, 2, 64)
    table = torch.zeros(2, 4, dtype=torch.int32)
    ctx = torch.zeros(2, dtype=torch.int32)
    f = fa_b200.flash_attention_decode_paged
    with pytest.raises(ValueError, match="paged query must be"):
        f(t(2, 4, 1, 64), kc, kc, table, ctx)
    with pytest.raises(ValueError, match="same shape"):
        f(q, kc, t(8, 16, 1, 64), table, ctx)
    with pytest.raises(ValueError, match="supported head dimension"):
        f(t(2, 4, 48), t(8, 16, 2, 48), t(8, 16, 2, 48), table, ctx)
    with pytest.raises(ValueError, match="multiple of cache heads"):
        f(t(2, 3, 64), kc, kc, table, ctx)
    with pytest.raises(ValueError, match="power of two"):
        f(q, t(8, 12, 2, 64), t(8, 12, 2, 64), table, ctx)
    with pytest.raises(ValueError, match="block_table must be an int32"):
        f(q, kc, kc, table.long(), ctx)
    with pytest.raises(ValueError, match="context_lens has an invalid shape"):
        f(q, kc, kc, table, ctx[:1])
    with pytest.raises(ValueError, match="max_context_len must be a nonnegative integer"):
        f(q, kc, kc, table, ctx, max_context_len=-1)
    with pytest.raises(ValueError, match="num_splits must be an integer between 1 and 32"):
        f(q, kc, kc, table, ctx, num_splits=33)
    with pytest.raises(RuntimeError, match="inference-only"):
        f(q.requires_grad_(True), kc, kc, table, ctx)
