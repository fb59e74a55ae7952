"""Host-side logic that needs no GPU: split heuristics, ALiBi slopes, op schemas with fake tensors, the
tiny-kernel routing predicate, and the SDPA dispatcher's routing, restoration and nesting
(modelled on the reference's tests/test_decode.py:38-43, tests/test_paged.py:172-179,
tests/test_torch_library.py, tests/test_sdpa_dispatch.py)."""
import threading

import pytest
import torch
import torch.nn.functional as F

import fa_b200
from fa_b200 import interface, sdpa


def test_decode_split_heuristic():
    f = interface._decode_num_splits
    assert f(1, 8, 1, 16384, 192) == 24
    assert f(4, 32, 1, 8192, 192) == 2
    assert f(4, 32, 1, 8192, 4 * 148) == 5          # the B200 call: 4 x 148 target programs
    assert f(1, 8, 1, 16384, 4 * 148) == 32         # capped at 32
    assert f(1, 1, 1, 100, 4 * 148) == 2            # never slices shorter than 64 keys
    assert f(64, 64, 1, 4096, 192) == 1


def test_paged_split_heuristic():
    f = interface._paged_num_splits
    assert f(1, 8, 16, 4, 96) == 1                                   # <= 64 tokens
    assert f(1, 8, 16, 16, 96) == 16
    # the reference's own table (tests/test_paged.py:172-179)
    assert f(1, 8, 16, 256, 96) == 16
    assert f(4, 32, 16, 256, 96, max_context_len=256) == 4
    assert f(8, 32, 16, 256, 96, max_context_len=256) == 2
    assert f(16, 32, 16, 256, 96, max_context_len=256) == 1
    assert f(16, 32, 16, 256, 96, max_context_len=4096) == 16
    assert f(4, 32, 16, 1024, 96, max_context_len=4096) == 16
    assert f(4, 32, 16, 1024, 2 * 148, max_context_len=16384) == 16   # headline paged configuration on B200
    assert f(4, 32, 16, 1024, 96, max_context_len=64) == 1
    assert f(4, 32, 16, 1024, 96, requested_splits=7) == 7


def test_b200_split_counts_fill_one_wave():
    """The B200 defaults (not the reference's 48-CU table): properties every launch relies on."""
    from fa_b200 import interface as I

    sm = 148
    # tensor-core split-K: even, one CTA per SM at most, at least two 128-key tiles per CTA
    for batch, kv_heads, seqlen_k in [(4, 32, 8192), (4, 8, 16384), (1, 8, 16384), (16, 32, 8192), (1, 1, 256), (2, 4, 100)]:
        s = I._decode_splits_b200(batch, kv_heads, 1, seqlen_k, sm, tensor_core=True)
        assert s >= 2 and s % 2 == 0
        assert batch * kv_heads * (s // 2) <= max(sm, batch * kv_heads)
        assert (s // 2) <= max(1, -(-seqlen_k // 128) // 2)
    assert I._decode_splits_b200(4, 32, 1, 16384, sm, tensor_core=True) == 2      # 128 CTAs already
    assert I._decode_splits_b200(1, 8, 1, 16384, sm, tensor_core=True) == 36      # 18 CTAs per head -> 144 CTAs
    # head dim 256: one partial per CTA, so the count is the CTA count (at least 2), still within one wave
    assert I._decode_splits_b200(4, 8, 4, 16384, sm, tensor_core=True, head_dim=256) == 4   # 32 heads x 4 = 128 CTAs
    assert I._decode_splits_b200(1, 8, 4, 16384, sm, tensor_core=True, head_dim=256) == 18  # 144 CTAs
    assert I._decode_splits_b200(4, 64, 4, 16384, sm, tensor_core=True, head_dim=256) == 2  # the kernel's minimum
    # tensor-core paged: one CTA row per batch entry, even count, CTAs within one wave
    s = I._paged_splits_b200(4, 8, 4, 16, 1024, sm, 16384, tensor_core=True)
    assert s == 74 and 4 * (s // 2) == 148
    s = I._paged_splits_b200(1, 8, 4, 16, 16, sm, 100, tensor_core=True)
    assert s == 6                                                                  # 100 tokens = 7 tiles: 3 CTAs of 2-3 tiles
    # CUDA-core kernels: slices of at least 512 keys (256 tokens paged), never more than 64 (32) of them
    for seqlen_k in (100, 512, 4096, 100000):
        s = I._decode_splits_b200(2, 4, 4, seqlen_k, sm)
        assert 1 <= s <= 64 and (s == 1 or seqlen_k // s >= 256)
    assert 1 <= I._paged_splits_b200(2, 4, 4, 16, 4096, sm) <= 32
    # the fill rule: fewest splits within 3 % of the fullest last wave, once there is one full wave
    assert I._fill_splits(32, 64, sm) == 18            # 576 CTAs on 296 slots: 97.3 % of two waves (37 would be 100 %: within 3 %)
    assert I._fill_splits(1000, 8, sm) == 2            # 2000 CTAs: 96.5 % of 7 waves, 12 points better than one split
    assert I._fill_splits(4, 64, sm, ctas_per_sm=1) == 37


def test_alibi_slopes_values_and_errors():
    s = fa_b200.alibi_slopes(8, device="cpu")
    assert torch.allclose(s, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s32 = fa_b200.alibi_slopes(32, device="cpu")
    assert torch.allclose(s32, torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)]))
    assert fa_b200.alibi_slopes(12, device="cpu").shape == (12,)
    for bad in (0, -1, 2.5, True):
        with pytest.raises(ValueError, match="positive integer"):
            fa_b200.alibi_slopes(bad, device="cpu")


def test_bias_is_expanded_not_materialised():
    q = torch.zeros(2, 4, 8, 16)
    bias = torch.zeros(1, 1, 8, 8)
    t, sbb, sbh, sbm, sbn, has = interface._bias_args(bias, q, 2, 4, 8, 8)
    assert has and (sbb, sbh) == (0, 0) and (sbm, sbn) == (8, 1) and t.data_ptr() == bias.data_ptr()
    assert interface._bias_args(None, q, 2, 4, 8, 8)[1:] == (0, 0, 0, 0, False)


def test_op_schemas_match_the_reference_surface():
    fwd = torch.ops.fa_b200.flash_fwd.default._schema
    bwd = torch.ops.fa_b200.flash_bwd.default._schema
    tiny = torch.ops.fa_b200.flash_tiny_fwd.default._schema
    assert [a.name for a in fwd.arguments] == ["query", "key", "value", "causal", "softmax_scale", "window_left",
                                               "window_right", "softcap", "bias", "alibi", "dropout_p", "dropout_seed"]
    assert [a.name for a in bwd.arguments][:6] == ["dout", "query", "key", "value", "out", "lse"]
    assert [a.name for a in tiny.arguments] == ["query", "key", "value", "softmax_scale", "bias", "block_n"]
    assert len(fwd.returns) == 2 and len(bwd.returns) == 3 and len(tiny.returns) == 1


def test_fake_tensor_rules():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(2, 8, 100, 64, dtype=torch.float16)
        k = torch.empty(2, 2, 130, 64, dtype=torch.float16)
        out, lse = torch.ops.fa_b200.flash_fwd(q, k, k, True, 0.125, -1, -1, 0.0, None, None, 0.0, 0)
        assert out.shape == q.shape and out.dtype == q.dtype
        assert lse.shape == (2, 8, 100) and lse.dtype == torch.float32
        dq, dk, dv = torch.ops.fa_b200.flash_bwd(out, q, k, k, out, lse, True, 0.125, -1, -1, 0.0, None, None, 0.0, 0)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape
        qv = torch.empty(300, 8, 64, dtype=torch.bfloat16)
        kv = torch.empty(300, 2, 64, dtype=torch.bfloat16)
        cu = torch.empty(4, dtype=torch.int32)
        o, l = torch.ops.fa_b200.varlen_fwd(qv, kv, kv, cu, cu, 128, 128, True, 0.125, -1, -1, 0.0, None)
        assert o.shape == qv.shape and l.shape == (8, 300)


def test_tiny_routing_predicate():
    q = torch.zeros(2, 8, 19, 128)
    ok = lambda **kw: interface._can_use_tiny_forward(
        kw.get("q", q), kw.get("k", q), q, kw.get("causal", False), kw.get("window", (-1, -1)), kw.get("softcap", 0.0),
        kw.get("alibi"), kw.get("dropout", 0.0), kw.get("q", q).shape[-1])
    assert ok()
    assert not ok(causal=True) and not ok(window=(3, 0)) and not ok(softcap=1.0) and not ok(dropout=0.1)
    assert not ok(alibi=torch.zeros(8))
    assert not ok(q=torch.zeros(2, 8, 33, 128), k=torch.zeros(2, 8, 33, 128))
    assert not ok(q=q.half())
    assert not ok(k=torch.zeros(2, 4, 19, 128))
    with torch.enable_grad():
        assert not ok(q=q.clone().requires_grad_(True))


# ------------------------------------------------------------------------------------------ SDPA dispatcher
@pytest.fixture
def spies(monkeypatch):
    calls = []
    monkeypatch.setattr(sdpa, "is_available", lambda device=None: True)
    monkeypatch.setattr(sdpa, "flash_attention", lambda q, k, v, **kw: calls.append(("flash", kw)) or q)
    monkeypatch.setattr(sdpa, "flash_attention_decode", lambda q, k, v, **kw: calls.append(("decode", kw)) or q)
    monkeypatch.setattr(sdpa, "_original_sdpa", lambda q, k, v, **kw: calls.append(("original", kw)) or q)

    class FakeCuda(torch.Tensor):
        is_cuda = True

    def cuda_like(*shape, dtype=torch.float16):
        return torch.zeros(*shape, dtype=dtype).as_subclass(FakeCuda)

    return calls, cuda_like


def test_dispatch_routes(spies):
    calls, t = spies
    q = t(2, 4, 128, 64)
    sdpa._dispatch_sdpa(q, q, q)
    assert calls[-1][0] == "flash" and calls[-1][1]["causal"] is False
    sdpa._dispatch_sdpa(q, q, q, is_causal=True, scale=0.2)
    assert calls[-1][0] == "flash" and calls[-1][1]["causal"] is True and calls[-1][1]["softmax_scale"] == 0.2
    # causal with different lengths: alignment differs from SDPA's top-left mask -> original
    sdpa._dispatch_sdpa(q, t(2, 4, 256, 64), t(2, 4, 256, 64), is_causal=True)
    assert calls[-1][0] == "original"
    sdpa._dispatch_sdpa(q, q, q, dropout_p=0.1)
    assert calls[-1][0] == "original"
    sdpa._dispatch_sdpa(q, t(2, 2, 128, 64), t(2, 2, 128, 64))
    assert calls[-1][0] == "original"                       # GQA needs enable_gqa=True
    sdpa._dispatch_sdpa(q, t(2, 2, 128, 64), t(2, 2, 128, 64), enable_gqa=True)
    assert calls[-1][0] == "flash"
    sdpa._dispatch_sdpa(t(2, 4, 128, 64, dtype=torch.float64), q, q)
    assert calls[-1][0] == "original"
    # decode route: short query, long cache, no mask, no grad
    sdpa._dispatch_sdpa(t(2, 4, 1, 64), t(2, 4, 2048, 64), t(2, 4, 2048, 64))
    assert calls[-1][0] == "decode"
    sdpa._dispatch_sdpa(t(2, 4, 1, 64), t(2, 4, 512, 64), t(2, 4, 512, 64))
    assert calls[-1][0] == "flash"


def test_dispatch_masks(spies):
    calls, t = spies
    q = t(1, 2, 16, 64)
    mask = torch.tensor([[True, False] * 8] * 16).as_subclass(type(q))
    sdpa._dispatch_sdpa(q, q, q, attn_mask=mask)
    bias = calls[-1][1]["bias"]
    assert calls[-1][0] == "flash" and bias.dtype == torch.float32
    assert torch.all(bias[:, 0::2] == 0) and torch.all(torch.isinf(bias[:, 1::2]))
    sdpa._dispatch_sdpa(q, q, q, attn_mask=mask, is_causal=True)
    assert calls[-1][0] == "original"
    sdpa._dispatch_sdpa(q, q, q, attn_mask=torch.zeros(3, 3).as_subclass(type(q)))
    assert calls[-1][0] == "original"


def test_dispatch_defers_tiny_training_shapes(spies):
    calls, t = spies
    q = t(1, 2, 12, 64).requires_grad_(True)
    sdpa._dispatch_sdpa(q, q, q)
    assert calls[-1][0] == "original"
    with torch.no_grad():
        sdpa._dispatch_sdpa(q, q, q)
    assert calls[-1][0] == "flash"


def test_bypass_is_thread_local(spies):
    calls, t = spies
    q = t(1, 2, 64, 64)
    seen = []
    with sdpa._bypass_flash_attention():
        sdpa._dispatch_sdpa(q, q, q)
        assert calls[-1][0] == "original"
        th = threading.Thread(target=lambda: (sdpa._dispatch_sdpa(q, q, q), seen.append(calls[-1][0])))
        th.start()
        th.join()
    assert seen == ["flash"]
    sdpa._dispatch_sdpa(q, q, q)
    assert calls[-1][0] == "flash"


def test_enable_disable_and_nested_context():
    original = F.scaled_dot_product_attention
    try:
        fa_b200.enable_flash_attention()
        assert F.scaled_dot_product_attention is sdpa._dispatch_sdpa
        fa_b200.enable_flash_attention()                       # idempotent
        fa_b200.disable_flash_attention()
        assert F.scaled_dot_product_attention is original
        with fa_b200.use_flash_attention():
            assert F.scaled_dot_product_attention is sdpa._dispatch_sdpa
            with fa_b200.use_rdna3_flash_attention():          # reference spelling, nests
                assert F.scaled_dot_product_attention is sdpa._dispatch_sdpa
            assert F.scaled_dot_product_attention is sdpa._dispatch_sdpa
        assert F.scaled_dot_product_attention is original
        fa_b200.enable_rdna3_flash_attention()
        with fa_b200.use_flash_attention():                    # context must not uninstall a global enable
            pass
        assert F.scaled_dot_product_attention is sdpa._dispatch_sdpa
    finally:
        fa_b200.disable_flash_attention()
        F.scaled_dot_product_attention = original


def test_unsupported_calls_fall_through_on_cpu():
    q = torch.randn(1, 2, 8, 16)
    with fa_b200.use_flash_attention():
        out = F.scaled_dot_product_attention(q, q, q)
    assert torch.allclose(out, F.scaled_dot_product_attention(q, q, q))


def test_wide_batch_pieces(monkeypatch):
    """Batch ranges for the scratch-buffer kernels of wide head dims: one range while the scratch fits its limit, else as
    many batch entries per launch as fit; never for widths or dtypes those kernels do not take."""
    from fa_b200 import interface as I

    q = torch.empty(6, 4, 300, 256, dtype=torch.float16)
    k = torch.empty(6, 2, 500, 256, dtype=torch.float16)
    per_entry = 2 * 4 * 3 * 4 * 32768                      # two tiles per 128 x 128 block, 4 heads, 3 x 4 blocks
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 6 * per_entry)
    assert I._wide_batch_pieces(q, k, 2, 128) == [(0, 6)]
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 2 * per_entry + 5)
    assert I._wide_batch_pieces(q, k, 2, 128) == [(0, 2), (2, 4), (4, 6)]
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 4 * per_entry)
    assert I._wide_batch_pieces(q, k, 2, 128) == [(0, 4), (4, 6)]
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", per_entry - 1)   # not even one entry: left to the caller
    assert I._wide_batch_pieces(q, k, 2, 128) == [(0, 6)]
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", per_entry)
    assert I._wide_batch_pieces(q[..., :128], k[..., :128], 2, 128) == [(0, 6)]            # fused kernels' width
    assert I._wide_batch_pieces(q.float(), k.float(), 2, 128) == [(0, 6)]                  # fp32 is never cut
    # forward scratch of head dims above 256: one tile per block plus 8 bytes per padded query row
    q5, k5 = torch.empty(3, 2, 256, 512, dtype=torch.bfloat16), torch.empty(3, 2, 256, 512, dtype=torch.bfloat16)
    monkeypatch.setattr(I, "DS_WORKSPACE_WIDE_LIMIT_BYTES", 2 * (2 * 2 * 32768 + 2 * 1024))
    assert I._wide_batch_pieces(q5, k5, 1, 256) == [(0, 1), (1, 2), (2, 3)]
