"""The ComfyUI adapter, exercised without ComfyUI: layout handling, fall-back rules, composition with an override that
was installed first, the model-patch node and the custom-node loader (the behaviours the reference checks in
tests/test_comfyui.py:16-312), plus GPU comparisons against torch SDPA through the adapter (:315-380 there)."""
import os
import subprocess
import sys

import pytest
import torch
import torch.nn.functional as F

from fa_b200 import comfyui, sdpa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _no_fallback(*args, **kwargs):
    raise AssertionError("the adapter fell back although the call is supported")


def _no_kernel(*args, **kwargs):
    raise AssertionError("the adapter called the kernels although the call must fall back")


class _Recorder:
    """Stands in for flash_attention: remembers what it was given and returns the query."""

    def __init__(self):
        self.calls = []

    def __call__(self, q, k, v, **kwargs):
        self.calls.append((q, k, v, kwargs))
        return q


@pytest.fixture
def kernels(monkeypatch):
    recorder = _Recorder()
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", recorder)
    return recorder


def test_token_layout_is_split_into_heads_and_restored(kernels):
    q, k, v = torch.randn(2, 5, 12), torch.randn(2, 7, 12), torch.randn(2, 7, 12)
    mask = torch.ones(5, 7, dtype=torch.bool)
    mask[:, -1] = False
    out = comfyui.ComfyUIAttentionOverride()(_no_fallback, q, k, v, 3, mask=mask, scale=0.25)
    (qh, kh, vh, kwargs), = kernels.calls
    assert qh.shape == (2, 3, 5, 4) and kh.shape == (2, 3, 7, 4) and vh.shape == (2, 3, 7, 4)
    # head h of token t is columns [4h, 4h + 4) of that token
    torch.testing.assert_close(qh[1, 2, 3], q[1, 3, 8:12])
    assert kwargs["softmax_scale"] == 0.25
    assert kwargs["bias"].shape == (1, 5, 7) and kwargs["bias"].dtype == torch.float32
    assert torch.all(kwargs["bias"][..., :-1] == 0) and torch.all(torch.isneginf(kwargs["bias"][..., -1]))
    torch.testing.assert_close(out, q)          # the recorder returns the query; the round trip restores the layout


def test_batched_mask_gets_a_head_dimension(kernels):
    q = torch.randn(2, 5, 8)
    mask = torch.zeros(2, 5, 5)
    comfyui.ComfyUIAttentionOverride()(_no_fallback, q, q, q, 2, mask=mask)
    assert kernels.calls[0][3]["bias"].shape == (2, 1, 5, 5)
    assert kernels.calls[0][3]["softmax_scale"] is None


def test_head_layout_with_grouped_kv_is_passed_through(kernels):
    q, k = torch.randn(2, 4, 5, 8), torch.randn(2, 2, 7, 8)
    out = comfyui.ComfyUIAttentionOverride()(_no_fallback, q, k, torch.randn_like(k), 4, skip_reshape=True,
                                            skip_output_reshape=True, enable_gqa=True)
    qh, kh, vh, _ = kernels.calls[0]
    assert qh is q and kh is k and vh.shape == k.shape
    assert out is q


def test_token_layout_with_grouped_kv(kernels):
    q, k = torch.randn(1, 5, 32), torch.randn(1, 7, 16)
    out = comfyui.ComfyUIAttentionOverride()(_no_fallback, q, k, k.clone(), 4, enable_gqa=True)
    assert kernels.calls[0][0].shape == (1, 4, 5, 8) and kernels.calls[0][1].shape == (1, 2, 7, 8)
    assert out.shape == (1, 5, 32)


@pytest.mark.parametrize("case", ["width", "rank", "batch", "kv_heads", "heads_type", "head_count"])
def test_shapes_that_do_not_describe_heads_fall_back(monkeypatch, case):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    q, k, v, heads, extra = torch.randn(2, 5, 12), torch.randn(2, 7, 12), torch.randn(2, 7, 12), 3, {}
    if case == "width":
        heads = 5
    elif case == "rank":
        q = q[0]
    elif case == "batch":
        k, v = k[:1], v[:1]
    elif case == "kv_heads":
        k, v = k[..., :4], v[..., :4]           # one kv head for three query heads, without enable_gqa
    elif case == "heads_type":
        heads = 3.0
    elif case == "head_count":
        q, k, v, extra = torch.randn(2, 4, 5, 4), torch.randn(2, 4, 7, 4), torch.randn(2, 4, 7, 4), {"skip_reshape": True}
    seen = {}

    def fallback(*args, **kwargs):
        seen["args"], seen["kwargs"] = args, kwargs
        return "fallback"

    assert comfyui.ComfyUIAttentionOverride()(fallback, q, k, v, heads, **extra) == "fallback"
    assert seen["args"][0] is q and seen["args"][3] == heads
    # the fall-back sees ComfyUI's own keywords, defaults filled in
    assert seen["kwargs"]["mask"] is None and seen["kwargs"]["skip_output_reshape"] is False
    assert seen["kwargs"]["skip_reshape"] is bool(extra)


def test_unsupported_call_falls_back_with_its_arguments(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: False)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    q = torch.randn(1, 4, 8)
    seen = {}

    def fallback(*args, **kwargs):
        seen.update(kwargs)
        return "fallback"

    out = comfyui.ComfyUIAttentionOverride()(fallback, q, q, q, 2, attn_precision=torch.float32, transformer_options={"x": 1})
    assert out == "fallback"
    assert seen["attn_precision"] == torch.float32 and seen["transformer_options"] == {"x": 1}


def test_requested_fp32_accumulation_falls_back_for_16_bit_inputs(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    q = torch.randn(1, 4, 8, dtype=torch.float16)
    out = comfyui.ComfyUIAttentionOverride()(lambda *a, **kw: "fallback", q, q, q, 2, attn_precision=torch.float32)
    assert out == "fallback"


def test_fp32_inputs_are_served_when_fp32_is_requested(kernels):
    q = torch.randn(1, 4, 8)
    comfyui.ComfyUIAttentionOverride()(_no_fallback, q, q, q, 2, attn_precision=torch.float32)
    assert len(kernels.calls) == 1


def test_precision_rule_of_the_host_application_is_consulted(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    asked = []

    def force_upcast(wanted, dtype):
        asked.append((wanted, dtype))
        return torch.float32

    q = torch.randn(1, 4, 8, dtype=torch.bfloat16)
    override = comfyui.ComfyUIAttentionOverride(precision_resolver=force_upcast)
    assert override(lambda *a, **kw: "fallback", q, q, q, 2) == "fallback"
    assert asked == [(None, torch.bfloat16)]


def test_low_precision_attention_false_falls_back(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    q = torch.randn(1, 4, 8)
    seen = {}

    def fallback(*args, **kwargs):
        seen.update(kwargs)
        return "fallback"

    assert comfyui.ComfyUIAttentionOverride()(fallback, q, q, q, 2, low_precision_attention=False) == "fallback"
    assert seen["low_precision_attention"] is False


def test_fallback_runs_with_the_sdpa_hook_bypassed(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: False)
    depths = []

    def fallback(*args, **kwargs):
        depths.append(getattr(sdpa._dispatch_bypass_state, "depth", 0))
        return "fallback"

    q = torch.randn(1, 4, 8)
    comfyui.ComfyUIAttentionOverride()(fallback, q, q, q, 2)
    assert depths == [1]
    assert getattr(sdpa._dispatch_bypass_state, "depth", 0) == 0


def test_earlier_override_is_called_first_and_may_answer_itself(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: True)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)
    seen = {}

    def earlier(attention, q, k, v, heads, **kwargs):
        seen["name"] = attention.__name__
        seen["kwargs"] = kwargs
        return "earlier"

    def comfy_attention(*args, **kwargs):
        raise AssertionError("not reached")

    q = torch.randn(1, 4, 8)
    out = comfyui.ComfyUIAttentionOverride(earlier)(comfy_attention, q, q, q, 2, scale=0.5)
    assert out == "earlier"
    assert seen["name"] == "comfy_attention"            # the delegate presents itself as the function it wraps
    assert seen["kwargs"]["scale"] == 0.5 and seen["kwargs"]["skip_reshape"] is False


def test_earlier_override_can_delegate_to_the_kernels(kernels):
    def add_one(attention, q, k, v, heads, **kwargs):
        return attention(q, k, v, heads, **kwargs) + 1

    q = torch.randn(2, 5, 12)
    out = comfyui.ComfyUIAttentionOverride(add_one)(_no_fallback, q, q, q, 3)
    assert len(kernels.calls) == 1 and kernels.calls[0][0].shape == (2, 3, 5, 4)
    torch.testing.assert_close(out, q + 1)


def test_earlier_override_delegating_an_unsupported_call_reaches_comfyui(monkeypatch):
    monkeypatch.setattr(comfyui, "_is_supported", lambda *args: False)
    monkeypatch.setattr(comfyui, "flash_attention", _no_kernel)

    def passes_on(attention, *args, **kwargs):
        return attention(*args, **kwargs)

    q = torch.randn(1, 4, 8)
    out = comfyui.ComfyUIAttentionOverride(passes_on)(lambda *a, **kw: ("comfy", kw["mask"]), q, q, q, 2)
    assert out == ("comfy", None)


class FakeModel:
    def __init__(self, transformer_options=None):
        self.model_options = {"transformer_options": dict(transformer_options or {})}
        self.clones = 0

    def clone(self):
        self.clones += 1
        return FakeModel(self.model_options["transformer_options"])


@pytest.fixture
def node_env(monkeypatch):
    enabled = []
    monkeypatch.setattr(comfyui, "unsupported_reason", lambda: None)
    monkeypatch.setattr(comfyui, "enable_flash_attention", lambda: enabled.append(True))
    monkeypatch.setattr(comfyui, "_get_comfyui_precision_resolver", lambda: (lambda wanted, dtype: wanted))
    return enabled


def test_node_patches_a_clone_and_switches_the_sdpa_hook_on(node_env):
    def earlier(attention, *args, **kwargs):
        return attention(*args, **kwargs)

    model = FakeModel({"optimized_attention_override": earlier, "other": 7})
    patched, = comfyui.ApplyB200FlashAttention().patch(model)
    assert patched is not model and model.clones == 1
    assert model.model_options["transformer_options"]["optimized_attention_override"] is earlier
    installed = patched.model_options["transformer_options"]["optimized_attention_override"]
    assert isinstance(installed, comfyui.ComfyUIAttentionOverride) and installed.previous_override is earlier
    assert patched.model_options["transformer_options"]["other"] == 7
    assert node_env == [True]
    # patching the patched model again keeps the adapter that is there
    again, = comfyui.ApplyB200FlashAttention().patch(patched)
    assert again.model_options["transformer_options"]["optimized_attention_override"] is installed


def test_node_on_a_model_without_an_override(node_env):
    patched, = comfyui.ApplyB200FlashAttention().patch(FakeModel())
    installed = patched.model_options["transformer_options"]["optimized_attention_override"]
    assert isinstance(installed, comfyui.ComfyUIAttentionOverride) and installed.previous_override is None


def test_node_refuses_an_unsupported_platform(monkeypatch):
    monkeypatch.setattr(comfyui, "unsupported_reason", lambda: "no sm_100 GPU")
    model = FakeModel()
    with pytest.raises(RuntimeError, match="no sm_100 GPU"):
        comfyui.ApplyB200FlashAttention().patch(model)
    assert model.clones == 0


def test_node_refuses_an_override_that_cannot_be_called(node_env):
    with pytest.raises(TypeError, match="must be callable"):
        comfyui.ApplyB200FlashAttention().patch(FakeModel({"optimized_attention_override": 3}))
    assert node_env == []


def test_node_tables():
    node = comfyui.NODE_CLASS_MAPPINGS["ApplyB200FlashAttention"]
    assert node is comfyui.ApplyB200FlashAttention
    assert comfyui.NODE_CLASS_MAPPINGS["ApplyRDNA3FlashAttention"] is node      # workflows saved for the reference
    assert set(comfyui.NODE_DISPLAY_NAME_MAPPINGS) == set(comfyui.NODE_CLASS_MAPPINGS)
    assert node.INPUT_TYPES() == {"required": {"model": ("MODEL",)}}
    assert node.RETURN_TYPES == ("MODEL",) and getattr(node, node.FUNCTION) is node.patch


_LOADER = """
import importlib.util, sys
sys.path.insert(0, {shadow!r})
{preload}
spec = importlib.util.spec_from_file_location("custom_node_under_test", {entry!r})
module = importlib.util.module_from_spec(spec)
spec.loader.exec_module(module)
import fa_b200
print(sorted(module.NODE_CLASS_MAPPINGS), fa_b200.__file__)
"""


def _run_loader(tmp_path, preload):
    shadow = tmp_path / "fa_b200"
    shadow.mkdir()
    (shadow / "__init__.py").write_text("SHADOW = True\n")
    entry = os.path.join(ROOT, "flash-attention-rdna3_b200", "__init__.py")
    code = _LOADER.format(shadow=str(tmp_path), preload=preload, entry=entry)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)


def test_custom_node_loader_prefers_the_package_beside_it(tmp_path):
    done = _run_loader(tmp_path, "")
    assert done.returncode == 0, done.stderr
    assert "ApplyB200FlashAttention" in done.stdout
    assert os.path.join("flash-attention-rdna3_b200", "fa_b200") in done.stdout


def test_custom_node_loader_refuses_a_foreign_package_that_is_already_loaded(tmp_path):
    done = _run_loader(tmp_path, "import fa_b200")
    assert done.returncode != 0
    assert "different fa_b200 package is already loaded" in done.stderr


# ---- on the GPU: the adapter end to end against torch SDPA ----

@pytest.mark.gpu
def test_token_layout_matches_sdpa_on_the_gpu():
    torch.manual_seed(7)
    heads, dim = 8, 64
    q = torch.randn(2, 300, heads * dim, device="cuda", dtype=torch.float16)
    k = torch.randn(2, 77, heads * dim, device="cuda", dtype=torch.float16)
    v = torch.randn_like(k)
    mask = torch.ones(2, 300, 77, dtype=torch.bool, device="cuda")
    mask[1, :, 60:] = False
    out = comfyui.ComfyUIAttentionOverride()(_no_fallback, q, k, v, heads, mask=mask)

    def split(t):
        return t.view(t.shape[0], t.shape[1], heads, dim).transpose(1, 2).float()

    want = F.scaled_dot_product_attention(split(q), split(k), split(v), attn_mask=mask.unsqueeze(1))
    want = want.transpose(1, 2).reshape(2, 300, heads * dim)
    torch.testing.assert_close(out.float(), want, atol=2e-3, rtol=2e-3)


@pytest.mark.gpu
def test_head_layout_with_grouped_kv_matches_sdpa_on_the_gpu():
    torch.manual_seed(8)
    q = torch.randn(2, 8, 256, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, 2, 512, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    out = comfyui.ComfyUIAttentionOverride()(_no_fallback, q, k, v, 8, skip_reshape=True, skip_output_reshape=True,
                                            enable_gqa=True, scale=0.11)
    want = F.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(4, 1), v.float().repeat_interleave(4, 1),
                                          scale=0.11)
    torch.testing.assert_close(out.float(), want, atol=1.6e-2, rtol=1.6e-2)


@pytest.mark.gpu
def test_fallback_does_not_come_back_through_the_sdpa_hook(monkeypatch):
    q = torch.randn(1, 2, 64, 32, device="cuda", dtype=torch.float16)
    want = F.scaled_dot_product_attention(q, q, q)
    monkeypatch.setattr(sdpa, "flash_attention", _no_kernel)

    def torch_attention(query, key, value, heads, **kwargs):
        return F.scaled_dot_product_attention(query, key, value)

    sdpa.enable_flash_attention()
    try:
        out = comfyui.ComfyUIAttentionOverride()(torch_attention, q, q, q, 2, skip_reshape=True,
                                                skip_output_reshape=True, low_precision_attention=False)
    finally:
        sdpa.disable_flash_attention()
    torch.testing.assert_close(out, want)
