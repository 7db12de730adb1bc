"""GPU tests at whole-model level on a seeded random-init multi-layer model with 4-bit projections,
a 4-bit embedding and a tied output projection:

  * the per-feature equivalence matrix -- greedy decode under each feature alone and under all of
    them against the unpatched model, tokens and logits (the reference's
    tests/test_model_equivalence.py:299-411 runs the same matrix on downloaded checkpoints; there are
    none here, so the model is random and the tolerance is the logit bound of `compile`);
  * reproducibility of the patched decode, bit for bit;
  * the timing harness that picks a feature plan;
  * a checkpoint directory written and read back gives bit-identical logits;
  * the output projection at vocabulary size (N = 128256) against the oracle.
"""

import json
import os

import pytest
import torch

from metile_b200 import backends as B
from metile_b200 import synth
from metile_b200.integrations import autotune, blocks, checkpoint, torch_lm
from oracle import affine as A
from oracle import cport
from tests.helpers import assert_bit_equal, assert_within

pytestmark = pytest.mark.gpu
TOLERANCE = 2e-2
FEATURE_SETS = {
    "attention": dict(attention=True, rms_norm=False, graph_fusion=False, quantized_mlp=False),
    "rms_norm": dict(attention=False, rms_norm=True, graph_fusion=False, quantized_mlp=False),
    "quantized_mlp": dict(attention=False, rms_norm=False, graph_fusion=False, quantized_mlp=True),
    "graph_fusion": dict(attention=False, rms_norm=False, graph_fusion=True, quantized_mlp=False),
    "everything": dict(attention=True, rms_norm=True, graph_fusion=True, quantized_mlp=True),
}
MATRIX = {}


def make_model(device):
    return blocks.random_model(seed=11, hidden=512, intermediate=1536, heads=8, kv_heads=2, head_dim=64, layers=4,
                               vocab=4096, device=device, tie_word_embeddings=True)


def prompt(device, batch=2):
    generator = torch.Generator().manual_seed(5)
    return torch.randint(1, 4096, (batch, 12), generator=generator).to(device)


@pytest.fixture(scope="module", autouse=True)
def write_matrix():
    yield
    out = os.environ.get("METILE_REPORT_DIR", "")
    if MATRIX and os.path.isdir(out):
        with open(os.path.join(out, "equivalence_matrix.json"), "w") as handle:
            json.dump(MATRIX, handle, indent=1, sort_keys=True)


@pytest.mark.parametrize("name", sorted(FEATURE_SETS))
def test_decode_matches_the_unpatched_model(cuda_device, name):
    model, tokens = make_model(cuda_device), prompt(cuda_device)
    steps = 8
    ref_tokens, ref_logits, _ = autotune.greedy_decode(model, tokens, steps)
    with torch_lm.apply_metile_to_torch_lm(model, **FEATURE_SETS[name]) as patch:
        assert patch.replacements, f"{name} patches nothing"
        got_tokens, got_logits, _ = autotune.greedy_decode(model, tokens, steps)
        refusals = dict(patch.refusals)
    valid, reason, same, diverged, relative = autotune.compare_decodes(
        (ref_tokens, ref_logits), (got_tokens, got_logits), TOLERANCE)
    MATRIX[name] = {"tokens_equal": same, "diverged_at": diverged, "logit_error_over_peak": relative,
                    "refusals": refusals}
    assert valid, reason
    after_tokens, after_logits, _ = autotune.greedy_decode(model, tokens, steps)
    assert after_tokens == ref_tokens and torch.equal(after_logits, ref_logits), "restore left something patched"


def test_patched_decode_is_reproducible(cuda_device):
    model, tokens = make_model(cuda_device), prompt(cuda_device)
    with torch_lm.apply_metile_to_torch_lm(model, **FEATURE_SETS["everything"]):
        first = autotune.greedy_decode(model, tokens, 6)
        second = autotune.greedy_decode(model, tokens, 6)
    assert first[0] == second[0]
    assert torch.equal(first[1], second[1]), "two patched runs differ bitwise"


def test_autotune_selects_a_verified_plan_and_caches_it(cuda_device):
    model, tokens = make_model(cuda_device), prompt(cuda_device, batch=1)
    plan = autotune.autotune_metile_for_torch_lm(model, tokens, decode_steps=6, trials=3)
    report = plan.report
    text = str(report)
    assert "unpatched:" in text and "selected:" in text
    assert len(report.measurements) == 15            # every non-empty subset of four features
    assert all(m.valid for m in report.measurements), [m.reason for m in report.measurements if not m.valid]
    if plan.feature_count:
        chosen = next(m for m in report.measurements if m.plan == plan)
        assert chosen.seconds_per_token < report.baseline_seconds_per_token
    assert autotune.autotune_metile_for_torch_lm(model, tokens, decode_steps=6, trials=3) is plan
    assert blocks.DecoderBlock.forward.__name__ == "forward", "the harness left a class patched"
    with plan.apply(model):
        autotune.greedy_decode(model, tokens, 2)
    out = os.environ.get("METILE_REPORT_DIR", "")
    if os.path.isdir(out):
        with open(os.path.join(out, "autotune_report.txt"), "w") as handle:
            handle.write(text + "\n")


@pytest.mark.parametrize("shards", [1, 2])
def test_checkpoint_round_trip_gives_identical_logits(cuda_device, tmp_path, shards):
    model, tokens = make_model(cuda_device), prompt(cuda_device)
    checkpoint.save_torch_lm(model, tmp_path, shards=shards)
    loaded = checkpoint.load_torch_lm(tmp_path, device=cuda_device)
    with torch.no_grad():
        assert_bit_equal(loaded(tokens), model(tokens), "logits of the reloaded model")
    with torch_lm.apply_metile_to_torch_lm(loaded, **FEATURE_SETS["everything"]):
        a = autotune.greedy_decode(loaded, tokens, 4)
        b = autotune.greedy_decode(model, tokens, 4)
    assert a[0] == b[0] and torch.equal(a[1], b[1])


@pytest.mark.parametrize("rows", [1, 16])
def test_output_projection_at_vocabulary_size(cuda_device, rows):
    """lm_head of Llama-3.2-1B: N = 128256 outputs over K = 2048, one and sixteen rows."""
    hidden, vocabulary = 2048, 128256
    weight = synth.affine_weight(31, vocabulary, hidden, cuda_device)
    x = synth.activations(32, rows, hidden, cuda_device, std=0.5)
    y = B.mlx_affine_qmv(x, *weight)
    packed, scales, biases = weight[0].cpu().numpy(), synth.to_numpy_bits(weight[1]), synth.to_numpy_bits(weight[2])
    reference = A.bf16_from_bits(cport.qmm(synth.to_numpy_bits(x), packed, scales, biases))
    assert_within(y, reference, what=f"lm_head {rows} rows")


def test_graphed_decoder_reproduces_the_eager_patched_decode(cuda_device):
    """One captured decode step replayed per token gives the tokens and the logits of the eager
    patched loop, bit for bit, and a second prompt through the same graph works as well."""
    from metile_b200.integrations.graphed import GraphedDecoder

    model, steps = make_model(cuda_device), 10
    with torch_lm.apply_metile_to_torch_lm(model, **FEATURE_SETS["everything"]) as patch:
        decoder = GraphedDecoder(model, batch=2, capacity=64)
        for seed in (5, 6):
            generator = torch.Generator().manual_seed(seed)
            tokens = torch.randint(1, 4096, (2, 12), generator=generator).to(cuda_device)
            eager_tokens, eager_logits, _ = autotune.greedy_decode(model, tokens, steps)
            first = decoder.prefill(tokens).argmax(dim=-1)
            generated = decoder.generate(first, steps)
            torch.cuda.synchronize()
            assert generated.t().tolist() == eager_tokens, f"prompt {seed}: tokens differ"
            assert torch.equal(decoder.logits, eager_logits[-1]), f"prompt {seed}: last logits differ"
            assert decoder.cache[0].length == 12 + steps
            assert decoder.cache[0].positions.tolist() == [12 + steps] * 2
        assert not patch.refusals, patch.refusals
