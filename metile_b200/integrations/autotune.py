"""Choose a feature plan for a model by timing its real decode loop.

The torch-side counterpart of `autotune_metile_for_mlx_lm` (metile/integrations/mlx_lm.py:3294-3530):
every subset of the requested features is applied in turn, its greedy decode is compared with the
unpatched model's (tokens and last-step logits, as tests/test_model_equivalence.py:299-411 compares
them), the subsets that reproduce the unpatched model are timed in interleaved rounds, and the
fastest one -- or no feature at all, when nothing beats the unpatched model -- is returned as a
plan.  Plans are remembered per model object, so a second call with the same arguments costs nothing.

What "reproduces" means here: the same greedy tokens, except that a first divergence is accepted
where the unpatched model's two best logits were closer than the logit tolerance (a tie the
rounding of either implementation may break either way); and last-step logits within `tolerance`
of the largest unpatched logit.  The fused kernels keep fp32 intermediates where the op-by-op model
rounds to bf16 after every projection, so bit-equal logits are not expected (the reference's tests
call this a reduction-order difference and bound it the same way).
"""

from __future__ import annotations

import itertools
import statistics
import time
import weakref
from dataclasses import dataclass, field

FEATURES = ("attention", "rms_norm", "graph_fusion", "quantized_mlp")


@dataclass(frozen=True)
class TorchLMPlan:
    """A measured feature combination (the fields `apply_metile_to_torch_lm` takes)."""

    attention: bool = False
    rms_norm: bool = False
    graph_fusion: bool = False
    quantized_mlp: bool = False
    report: object = field(default=None, compare=False, repr=False, hash=False)

    @property
    def flags(self):
        return {name: getattr(self, name) for name in FEATURES}

    @property
    def feature_count(self):
        return sum(self.flags.values())

    def apply(self, model):
        """Patch `model` with this plan; returns the reversible handle."""
        from .torch_lm import apply_metile_to_torch_lm

        return apply_metile_to_torch_lm(model, **self.flags)


@dataclass
class PlanMeasurement:
    plan: TorchLMPlan
    valid: bool
    reason: str = ""
    tokens_match: bool = True
    diverged_at: int | None = None
    logit_relative: float = 0.0
    patched: tuple = ()
    seconds_per_token: float | None = None
    samples: list = field(default_factory=list)


@dataclass
class PlanReport:
    selected: TorchLMPlan
    baseline_seconds_per_token: float
    measurements: list
    decode_steps: int
    trials: int

    def __str__(self):
        lines = [f"unpatched: {self.baseline_seconds_per_token * 1e6:.1f} us per token "
                 f"({self.decode_steps} decode steps, median of {self.trials} interleaved rounds)"]
        for m in sorted(self.measurements, key=lambda m: (m.seconds_per_token is None, m.seconds_per_token or 0.0)):
            names = "+".join(name for name, on in m.plan.flags.items() if on) or "(none)"
            if m.valid:
                lines.append(f"  {names}: {m.seconds_per_token * 1e6:.1f} us per token, logits within "
                             f"{m.logit_relative:.1e}, tokens {'equal' if m.tokens_match else f'tie at step {m.diverged_at}'}")
            else:
                lines.append(f"  {names}: rejected, {m.reason}")
        chosen = "+".join(name for name, on in self.selected.flags.items() if on) or "(none)"
        lines.append(f"selected: {chosen}")
        return "\n".join(lines)


def _logits_of(output):
    return getattr(output, "logits", output)


def greedy_decode(model, tokens, steps):
    """Prefill `tokens` [B, T], then `steps` greedy decode steps with the model's own cache.

    Returns (generated tokens, one list per step with the prefill's token first; the logits
    [steps + 1, B, V] each of those tokens was the argmax of, as float32; the seconds the decode steps
    took on the device -- prefill not included)."""
    import torch

    batch, length = tokens.shape
    with torch.no_grad():
        make_cache = getattr(model, "make_cache", None)
        if make_cache is None:
            raise TypeError("the model must offer make_cache(batch, capacity) for a decode loop")
        cache = make_cache(batch, length + steps + 1)
        out = _logits_of(model(tokens, cache=cache))
        following = out[:, -1, :].argmax(dim=-1)
        generated, logits = [following.tolist()], [out[:, -1, :].float()]
        on_device = tokens.is_cuda
        if on_device:
            torch.cuda.synchronize(tokens.device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        begin = time.perf_counter()
        for _ in range(steps):
            out = _logits_of(model(following[:, None], cache=cache))
            following = out[:, -1, :].argmax(dim=-1)
            logits.append(out[:, -1, :].float())
            generated.append(following)
        if on_device:
            stop.record()
            torch.cuda.synchronize(tokens.device)
            seconds = start.elapsed_time(stop) * 1e-3
        else:
            seconds = time.perf_counter() - begin
        generated = [generated[0]] + [step.tolist() for step in generated[1:]]
        return generated, torch.stack(logits), seconds


def compare_decodes(reference, candidate, tolerance):
    """(valid, reason, tokens_match, diverged_at, logit_relative) of a candidate decode against the
    unpatched one; both are (tokens, logits) as `greedy_decode` returns them."""
    ref_tokens, ref_logits = reference
    got_tokens, got_logits = candidate
    import torch

    if not torch.isfinite(got_logits).all():
        return False, "non-finite logits", False, None, float("inf")
    peak = float(ref_logits.abs().max())
    diverged = next((i for i, (a, b) in enumerate(zip(ref_tokens, got_tokens)) if a != b), None)
    # Logits are comparable step by step only while both runs have seen the same tokens:
    # generated[d] is the argmax of logits[d], so logits[0 .. d] had identical inputs.
    comparable = ref_logits.shape[0] if diverged is None else diverged + 1
    relative = 0.0
    if comparable and peak > 0:
        relative = float((got_logits[:comparable] - ref_logits[:comparable]).abs().max()) / peak
    if relative > tolerance:
        return False, f"logits differ by {relative:.2e} of the largest logit (tolerance {tolerance:.1e})", diverged is None, diverged, relative
    if diverged is not None:
        # A tie in the logits the diverging token was chosen from may break either way.
        row = ref_logits[diverged]
        top = row.topk(2, dim=-1).values
        margin = float((top[..., 0] - top[..., 1]).min())
        if margin > 2 * tolerance * peak:
            return False, (f"greedy tokens diverge at step {diverged} where the unpatched margin {margin:.3g} "
                           f"is not a tie"), False, diverged, relative
        return True, "", False, diverged, relative
    return True, "", True, None, relative


_plans = weakref.WeakKeyDictionary()


def _candidates(requested):
    names = [name for name in FEATURES if requested[name]]
    subsets = []
    for size in range(1, len(names) + 1):
        for chosen in itertools.combinations(names, size):
            subsets.append(TorchLMPlan(**{name: name in chosen for name in FEATURES}))
    return subsets


def autotune_metile_for_torch_lm(model, sample_tokens, *, attention=True, rms_norm=True, graph_fusion=True,
                                 quantized_mlp=True, decode_steps=8, trials=5, tolerance=2e-2, margin=0.02):
    """Measure every subset of the requested features on `model`'s decode loop and return the
    fastest one that reproduces the unpatched model (a `TorchLMPlan`; `.report` holds the table).
    A plan must beat the unpatched model by `margin` to be preferred over patching nothing."""
    from .torch_lm import apply_metile_to_torch_lm

    if not callable(model):
        raise TypeError("model must be a callable torch module")
    if sample_tokens.ndim != 2 or sample_tokens.shape[1] < 1:
        raise ValueError("sample_tokens must have shape [batch, sequence]")
    if decode_steps < 1 or trials < 1:
        raise ValueError("decode_steps and trials must be positive")
    requested = {"attention": bool(attention), "rms_norm": bool(rms_norm), "graph_fusion": bool(graph_fusion),
                 "quantized_mlp": bool(quantized_mlp)}
    key = (tuple(sample_tokens.shape), tuple(requested.items()), decode_steps, trials, tolerance)
    cached = _plans.get(model, {}).get(key)
    if cached is not None:
        return cached

    ref_tokens, ref_logits, _ = greedy_decode(model, sample_tokens, decode_steps)
    reference = (ref_tokens, ref_logits)
    measurements = []
    for plan in _candidates(requested):
        with apply_metile_to_torch_lm(model, **plan.flags) as patch:
            patched = tuple(sorted({getattr(owner, "__name__", str(owner)) for owner, _, _ in patch.replacements}))
            if not patched:
                measurements.append(PlanMeasurement(plan, False, "patches nothing on this model"))
                continue
            tokens, logits, _ = greedy_decode(model, sample_tokens, decode_steps)
        valid, reason, same, diverged, relative = compare_decodes(reference, (tokens, logits), tolerance)
        measurements.append(PlanMeasurement(plan, valid, reason, same, diverged, relative, patched))

    # Interleaved rounds: every candidate once per round, so drift hits all of them alike.
    baseline_samples = []
    runnable = [m for m in measurements if m.valid]
    for _ in range(trials):
        baseline_samples.append(greedy_decode(model, sample_tokens, decode_steps)[2] / decode_steps)
        for m in runnable:
            with apply_metile_to_torch_lm(model, **m.plan.flags):
                m.samples.append(greedy_decode(model, sample_tokens, decode_steps)[2] / decode_steps)
    baseline = statistics.median(baseline_samples)
    for m in runnable:
        m.seconds_per_token = statistics.median(m.samples)

    best = min(runnable, key=lambda m: m.seconds_per_token, default=None)
    if best is not None and best.seconds_per_token < baseline * (1.0 - margin):
        flags = best.plan.flags
    else:
        flags = {name: False for name in FEATURES}
    report = PlanReport(TorchLMPlan(**flags), baseline, measurements, decode_steps, trials)
    selected = TorchLMPlan(**flags, report=report)
    report.selected = selected
    _plans.setdefault(model, {})[key] = selected
    return selected
