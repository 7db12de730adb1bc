"""CPU tests of the patcher and of `compile`: report semantics, structural admission, restore,
per-call refusal, bisecting.  The CUDA operators are replaced by torch stand-ins, in the way the
reference's patcher tests replace kernels with recording fakes
(tests/test_mlx_backend.py:3184-3558, tests/test_compile.py:18-94 of the reference)."""

import pytest
import torch
from torch import nn

import metile_b200
from metile_b200 import backends
from metile_b200.compile import CompileReport
from metile_b200.integrations import torch_lm


class FakeQuantizedLinear(nn.Module):
    """Carries the attributes the support gate inspects; computes with a dense float weight."""

    def __init__(self, fan_in, fan_out, seed, bias=False, bits=4):
        super().__init__()
        generator = torch.Generator().manual_seed(seed)
        self.dense = (torch.randn((fan_out, fan_in), generator=generator) / fan_in ** 0.5).to(torch.bfloat16)
        self.weight = torch.zeros((fan_out, fan_in // 8), dtype=torch.int32)
        self.scales = torch.ones((fan_out, fan_in // 64), dtype=torch.bfloat16)
        self.biases = torch.zeros((fan_out, fan_in // 64), dtype=torch.bfloat16)
        self.group_size, self.bits, self.mode = 64, bits, "affine"
        self.bias = torch.zeros(fan_out, dtype=torch.bfloat16) if bias else None

    def forward(self, values):
        return (values.float() @ self.dense.float().t()).to(values.dtype)


class FakeNorm(nn.Module):
    def __init__(self, width):
        super().__init__()
        self.weight = torch.ones(width, dtype=torch.bfloat16)
        self.eps = 1e-6

    def forward(self, values):
        v = values.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(values.dtype)


class FakeMLP(nn.Module):
    def __init__(self, width, inter, seed, **kw):
        super().__init__()
        self.gate_proj = FakeQuantizedLinear(width, inter, seed, **kw)
        self.up_proj = FakeQuantizedLinear(width, inter, seed + 1, **kw)
        self.down_proj = FakeQuantizedLinear(inter, width, seed + 2, **kw)

    def forward(self, values):
        return self.down_proj(nn.functional.silu(self.gate_proj(values)) * self.up_proj(values))


class FakeAttention(nn.Module):
    def forward(self, values, cache=None):
        return values * 0.5


class FakeBlock(nn.Module):
    def __init__(self, width, inter, seed, **kw):
        super().__init__()
        self.input_layernorm, self.post_attention_layernorm = FakeNorm(width), FakeNorm(width)
        self.self_attn, self.mlp = FakeAttention(), FakeMLP(width, inter, seed, **kw)

    def forward(self, values, cache=None):
        hidden = values + self.self_attn(self.input_layernorm(values), cache)
        return hidden + self.mlp(self.post_attention_layernorm(hidden))


class FakeLM(nn.Module):
    def __init__(self, width=64, inter=128, vocab=50, layers=2, **kw):
        super().__init__()
        self.vocab_size = vocab
        generator = torch.Generator().manual_seed(5)
        self.table = torch.randn((vocab, width), generator=generator).to(torch.bfloat16)
        self.layers = nn.ModuleList([FakeBlock(width, inter, 10 * i, **kw) for i in range(layers)])
        self.norm = FakeNorm(width)
        self.head = torch.randn((vocab, width), generator=generator).to(torch.bfloat16)

    def make_cache(self):
        return [None for _ in self.layers]

    def forward(self, tokens, cache=None):
        hidden = self.table[tokens]
        for layer in self.layers:
            hidden = layer(hidden)
        return (self.norm(hidden).float() @ self.head.float().t())


@pytest.fixture
def fake_kernels(monkeypatch):
    """torch stand-ins for the CUDA operators, recording calls; `skew` perturbs the fused MLP."""
    calls = {"mlp": 0, "add_rms": 0, "rms": 0, "skew": 0.0}

    def fake_executor(sample, gw, gs, gb, uw, us, ub, dw, ds, db, sample_residual, **_):
        def execute(values, residual=None):
            calls["mlp"] += 1
            module = fake_executor.module
            out = module.down_proj(nn.functional.silu(module.gate_proj(values)) * module.up_proj(values))
            out = out.float() * (1.0 + calls["skew"])
            if residual is not None:
                out = out + residual.float()
            return out.to(values.dtype)

        return execute

    def fake_execute_quantized_mlp(module, values, residual=None):
        fake_executor.module = module
        return fake_executor(values, *[None] * 9, None)(values, residual)

    def fake_add_rms(values, residual, weight, eps, **_):
        calls["add_rms"] += 1
        total = values + residual
        v = total.float()
        return total, (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(values.dtype)

    def fake_rms(values, weight, eps, **_):
        calls["rms"] += 1
        v = values.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(values.dtype)

    monkeypatch.setattr(torch_lm, "execute_quantized_mlp", fake_execute_quantized_mlp)
    monkeypatch.setattr(backends, "mlx_add_rms_norm", fake_add_rms)
    monkeypatch.setattr(backends, "mlx_rms_norm", fake_rms)
    # The gate refuses CPU tensors; the fakes run on CPU, so relax only that clause.
    original_gate = torch_lm.quantized_mlp_refusal

    def cpu_gate(module, values):
        reason = original_gate(module, values)
        return None if reason == "activations are not on a CUDA device" else reason

    monkeypatch.setattr(torch_lm, "quantized_mlp_refusal", cpu_gate)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    return calls


def test_report_truthiness_and_wording():
    empty = CompileReport(model="llama")
    assert not empty
    assert "accelerating: nothing" in str(empty)
    kept = CompileReport(model="qwen2", features=("rms_norm",), surfaces=("input_layernorm",), verified=True,
                         difference=0.0)
    assert kept and "logits match the unpatched model exactly" in str(kept)
    close = CompileReport(model="llama", features=("quantized_mlp",), surfaces=("mlp",), verified=True,
                          difference=0.0352, relative=2.3e-3, declined={"attention": "no kernel"})
    text = str(close)
    assert "within tolerance, logits differ by 0.0352 (2.3e-03 relative)" in text
    assert "declined attention: no kernel" in text
    assert "skipped (verify=False)" in str(CompileReport(model="x", features=("rms_norm",), verified=None))
    assert "FAILED, everything reverted" in str(CompileReport(model="x", verified=False))


def test_compile_rejects_non_models():
    with pytest.raises(TypeError):
        metile_b200.compile(None)
    with pytest.raises(TypeError):
        metile_b200.compile(3)


def test_compile_patches_verifies_and_restores(fake_kernels):
    model = FakeLM()
    original_block, original_mlp, original_norm = FakeBlock.forward, FakeMLP.forward, FakeNorm.forward
    report = metile_b200.compile(model, tolerance=1e-2)
    try:
        assert report and report.verified is True
        assert set(report.features) == {"rms_norm", "graph_fusion", "quantized_mlp"}
        assert "block" in report.surfaces and "mlp" in report.surfaces
        assert "attention" in report.declined  # asked for, no kernel: recorded, not silently dropped
        assert FakeBlock.forward._metile_original is original_block
        assert fake_kernels["mlp"] > 0 and fake_kernels["add_rms"] > 0 and fake_kernels["rms"] > 0
    finally:
        report.restore()
    assert FakeBlock.forward is original_block and FakeMLP.forward is original_mlp
    assert FakeNorm.forward is original_norm
    report.restore()  # idempotent


def test_compile_bisects_and_declines_a_wrong_surface(fake_kernels):
    model = FakeLM()
    fake_kernels["skew"] = 0.5  # the fused MLP now computes something else
    report = metile_b200.compile(model, tolerance=1e-2)
    try:
        assert "combined" in report.declined
        assert "quantized_mlp" in report.declined and "different computation" in report.declined["quantized_mlp"]
        # Block fusion alone calls the module's own MLP, so it still reproduces the logits.
        assert report.features == ("rms_norm", "graph_fusion")
    finally:
        report.restore()
    assert not hasattr(FakeMLP.forward, "_metile_original")


def test_reduction_order_scale_wording(fake_kernels):
    model = FakeLM()
    fake_kernels["skew"] = 2e-3
    report = metile_b200.compile(model, tolerance=0.0, features=("quantized_mlp",))
    try:
        assert not report
        assert report.verified is False
        assert "reduction-order scale, raise tolerance to keep it" in report.declined["quantized_mlp"]
    finally:
        report.restore()


def test_unsupported_projection_is_refused_per_call_not_rerouted(fake_kernels):
    model = FakeLM(bias=True)  # additive bias: outside the kernels' format
    report = metile_b200.compile(model, tolerance=1e-2, features=("quantized_mlp", "graph_fusion"))
    try:
        assert fake_kernels["mlp"] == 0  # the original forward served every call
        assert "quantized_mlp" in report.declined and "additive bias" in report.declined["quantized_mlp"]
        assert "quantized_mlp" not in report.features
    finally:
        report.restore()


def test_model_without_replaceable_classes_reports_nothing():
    class Plain(nn.Module):
        vocab_size = 11

        def forward(self, tokens, cache=None):
            return torch.zeros((*tokens.shape, 11))

    report = metile_b200.compile(Plain())
    assert not report
    assert "surfaces" in report.declined


def test_row_gates_and_handle_context_manager(fake_kernels):
    model = FakeLM()
    with torch_lm.apply_metile_to_torch_lm(model, graph_fusion=False, rms_norm=False, quantized_mlp=True,
                                           quantized_mlp_min_rows=4, quantized_mlp_max_rows=8) as patch:
        x = torch.randn((1, 2, 64)).to(torch.bfloat16)
        model.layers[0].mlp(x)
        assert fake_kernels["mlp"] == 0  # 2 rows < min_rows
        model.layers[0].mlp(torch.randn((1, 6, 64)).to(torch.bfloat16))
        assert fake_kernels["mlp"] == 1
        model.layers[0].mlp(torch.randn((1, 16, 64)).to(torch.bfloat16))
        assert fake_kernels["mlp"] == 1  # 16 rows > max_rows
        assert patch.replacements
    assert not hasattr(FakeMLP.forward, "_metile_original")
    with pytest.raises(ValueError):
        torch_lm.apply_metile_to_torch_lm(model, quantized_mlp_min_rows=0)
    # A refused call leaves nothing patched behind.
    assert not hasattr(FakeBlock.forward, "_metile_original") and not hasattr(FakeMLP.forward, "_metile_original")
    with pytest.raises(ValueError):
        torch_lm.apply_metile_to_torch_lm(None)


def test_structural_detection_excludes_as_well_as_admits():
    """Structure has to exclude as well as admit (the reference's tests/test_compile.py:55-77): an
    attention class is not a gated MLP, an MLP is not a decoder block, a norm is neither."""
    from metile_b200.integrations import blocks

    mlp_parts, block_parts = torch_lm._GATED_MLP_ATTRIBUTES, torch_lm._FUSED_BLOCK_ATTRIBUTES
    for mlp_class in (FakeMLP, blocks.GatedMLP):
        assert torch_lm._structurally_matches(mlp_class, mlp_parts)
        assert not torch_lm._structurally_matches(mlp_class, block_parts)
    for block_class in (FakeBlock, blocks.DecoderBlock):
        assert torch_lm._structurally_matches(block_class, block_parts)
        assert not torch_lm._structurally_matches(block_class, mlp_parts)
    for other in (FakeAttention, blocks.Attention, FakeNorm, blocks.RMSNorm, FakeQuantizedLinear):
        assert not torch_lm._structurally_matches(other, mlp_parts)
        assert not torch_lm._structurally_matches(other, block_parts)
    assert torch_lm._structurally_matches(FakeNorm, ("weight",))

    class DeclaredParts(nn.Module):
        """Parts declared on the class rather than bound in __init__ are seen as well."""

        gate_proj: nn.Module
        up_proj: nn.Module
        down_proj: nn.Module

        def forward(self, values):
            return values

    assert torch_lm._structurally_matches(DeclaredParts, mlp_parts)


def test_structural_detection_needs_a_forward_to_replace():
    """A class that defines no forward of its own has nothing to swap (tests/test_compile.py:80-94 of
    the reference): nn.Module's inherited placeholder does not count."""

    class HasThePartsButNoForward(nn.Module):
        gate_proj = up_proj = down_proj = staticmethod(lambda x: x)

    assert not torch_lm._structurally_matches(HasThePartsButNoForward, torch_lm._GATED_MLP_ATTRIBUTES)

    class InheritsForward(FakeMLP):
        pass

    assert torch_lm._structurally_matches(InheritsForward, torch_lm._GATED_MLP_ATTRIBUTES)


def test_an_attention_class_in_the_mlp_slot_is_not_patched(fake_kernels):
    """A layer whose `mlp` is not a gated MLP keeps its own forward and `compile` says so."""
    model = FakeLM()
    for layer in model.layers:
        layer.mlp = FakeAttention()
    handle = torch_lm.apply_metile_to_torch_lm(model=model, rms_norm=False, graph_fusion=False, quantized_mlp=True)
    try:
        assert handle.replacements == []
        assert getattr(FakeAttention.forward, "_metile_original", None) is None
    finally:
        handle.restore()


def test_survivors_of_the_bisection_are_kept_together(fake_kernels):
    """When the full set disagrees, the features that verify alone are applied together."""
    fake_kernels["skew"] = 0.25  # the fused MLP is wrong; the norms are right
    model = FakeLM()
    report = metile_b200.compile(model, features=("rms_norm", "quantized_mlp"))
    try:
        assert report.features == ("rms_norm",)
        assert "quantized_mlp" in report.declined and "combined" in report.declined
        assert report.verified is True and report.difference == 0.0
    finally:
        report.restore()


def test_attention_patch_replaces_the_module_level_primitive_and_restores_it():
    """The attention feature swaps the `scaled_dot_product_attention` attribute of the module that
    defines the model's attention class (as the reference swaps mlx_lm.models.base's) and the class's
    forward; a call the kernel cannot serve (here: CPU tensors) is passed on and recorded."""
    from metile_b200.integrations import blocks

    model = blocks.random_model(seed=1, hidden=64, intermediate=128, heads=2, kv_heads=1, head_dim=64, layers=1,
                                vocab=32, device="cpu")
    original_sdpa, original_forward = blocks.scaled_dot_product_attention, blocks.Attention.forward
    with torch_lm.apply_metile_to_torch_lm(model, attention=True, rms_norm=False, graph_fusion=False,
                                           quantized_mlp=False) as patch:
        assert blocks.scaled_dot_product_attention._metile_original is original_sdpa
        assert blocks.Attention.forward._metile_original is original_forward
        q = torch.randn((1, 2, 1, 64)).to(torch.bfloat16)
        kv = torch.randn((1, 1, 5, 64)).to(torch.bfloat16)
        out = blocks.scaled_dot_product_attention(q, kv, kv, None, 0.125, None)
        assert out.shape == (1, 2, 1, 64)
        assert "attention" in patch.refusals and "CUDA" in patch.refusals["attention"]
        prefill = blocks.scaled_dot_product_attention(torch.randn((1, 2, 5, 64)).to(torch.bfloat16), kv, kv, None, 0.125,
                                                      "causal")
        assert prefill.shape == (1, 2, 5, 64)
    assert blocks.scaled_dot_product_attention is original_sdpa and blocks.Attention.forward is original_forward
    # A model without an attention surface says so instead of silently keeping the feature.
    with torch_lm.apply_metile_to_torch_lm(FakeLM(), attention=True, rms_norm=False, graph_fusion=False,
                                           quantized_mlp=False) as patch:
        assert "no attention surface" in patch.refusals["attention"]


def test_autotune_argument_checks_and_cpu_run():
    """On the CPU every patched call refuses and falls back to the model's own code, so every subset
    reproduces the unpatched model exactly; the harness still compares, times and reports them."""
    from metile_b200.integrations import autotune, blocks

    with pytest.raises(TypeError):
        autotune.autotune_metile_for_torch_lm(object(), torch.zeros((1, 4), dtype=torch.long))
    lm = FakeLM()
    with pytest.raises(ValueError):
        autotune.autotune_metile_for_torch_lm(lm, torch.zeros((4,), dtype=torch.long))
    with pytest.raises(ValueError):
        autotune.autotune_metile_for_torch_lm(lm, torch.zeros((1, 4), dtype=torch.long), decode_steps=0)
    assert blocks.DecoderBlock.forward.__name__ == "forward"  # nothing left patched by the refusals above


def test_compare_decodes_accepts_ties_and_rejects_real_divergence():
    from metile_b200.integrations.autotune import compare_decodes

    logits = torch.tensor([[[5.0, 4.999, 0.0]], [[1.0, 9.0, 0.0]]])       # step 0 is a near tie, step 1 is not
    same = ([[0], [1]], logits)
    assert compare_decodes(same, same, 1e-2)[:3] == (True, "", True)
    tie = ([[1], [1]], logits.clone())                                     # diverges at generated[0], a tie
    valid, reason, match, at, _ = compare_decodes(same, tie, 1e-2)
    assert valid and not match and at == 0
    real = ([[0], [2]], logits.clone())                                    # diverges where the margin is 8
    valid, reason, match, at, _ = compare_decodes(same, real, 1e-2)
    assert not valid and at == 1 and "not a tie" in reason
    off = (same[0], logits + torch.tensor(1.0))
    valid, reason, *_ = compare_decodes(same, off, 1e-2)
    assert not valid and "logits differ" in reason
    assert not compare_decodes(same, (same[0], logits * float("nan")), 1e-2)[0]
