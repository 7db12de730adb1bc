"""One call that accelerates a torch model carrying MLX INT4 weights and reports what it did.

torch-side equivalent of the reference's `metile.compile` (metile/compile.py:146-254) with the
same contract:
  * candidates are admitted by structure, then VERIFIED: the model runs before and after
    patching (a prefill and four greedy decode steps, last-step logits in float32,
    compile.py:97-115) and the logits are compared; if the whole feature set disagrees it is
    bisected one feature at a time (compile.py:203-233);
  * `tolerance` is relative to the largest reference logit and defaults to exact; about 5e-3 is
    the scale of a summation reorder (REORDERING_SCALE, compile.py:48);
  * the report is falsy when nothing was replaced, names the replaced surfaces, and lists every
    declined feature with its reason -- including per-call refusals of the patched surfaces
    (a call the kernels cannot serve runs the original forward; it is never rerouted silently).
"""

from __future__ import annotations

from dataclasses import dataclass, field

FEATURES = ("attention", "rms_norm", "graph_fusion", "quantized_mlp")
TOLERANCE = 0.0
REORDERING_SCALE = 5e-3


@dataclass
class CompileReport:
    """What `compile` replaced, what it declined, and why."""

    model: str = "unknown"
    features: tuple = ()
    surfaces: tuple = ()
    verified: bool | None = None
    difference: float | None = None
    relative: float | None = None
    declined: dict = field(default_factory=dict)
    handle: object = None

    def __bool__(self):
        """False when nothing was replaced, so `if not compile(model)` is a usable check."""
        return bool(self.features)

    def restore(self):
        """Put back the model's own implementations."""
        if self.handle is not None:
            self.handle.__exit__(None, None, None)
            self.handle = None

    def __str__(self):
        lines = [f"meTile on {self.model}"]
        if self.features:
            lines.append(f"  accelerating: {', '.join(self.features)}")
            lines.append(f"  surfaces replaced: {', '.join(self.surfaces) or 'none reported'}")
        else:
            lines.append("  accelerating: nothing -- this model runs entirely on its own implementations")
        if self.verified is None:
            lines.append("  verification: skipped (verify=False)")
        elif self.verified and not self.difference:
            lines.append("  verification: logits match the unpatched model exactly")
        elif self.verified:
            lines.append(
                f"  verification: within tolerance, logits differ by {self.difference:g}"
                + (f" ({self.relative:.1e} relative)" if self.relative else "")
            )
        else:
            lines.append("  verification: FAILED, everything reverted")
        for feature, reason in sorted(self.declined.items()):
            lines.append(f"  declined {feature}: {reason}")
        return "\n".join(lines)


def _logits_of(output):
    return getattr(output, "logits", output)


def _decode_logits(model, tokens, steps=4):
    """Prefill, take a few greedy decode steps, return the last step's logits as float32.

    Decode steps rather than prefill only, so that the one-row kernels are exercised too."""
    import torch

    with torch.no_grad():
        make_cache = getattr(model, "make_cache", None)
        if make_cache is not None:
            cache = make_cache()
            out = _logits_of(model(tokens, cache=cache))
            following = out[:, -1, :].argmax(dim=-1)
            for _ in range(steps):
                out = _logits_of(model(following[:, None], cache=cache))
                following = out[:, -1, :].argmax(dim=-1)
            return out[:, -1, :].float()
        sequence = tokens
        out = _logits_of(model(sequence))
        for _ in range(steps):
            following = out[:, -1, :].argmax(dim=-1)
            sequence = torch.cat([sequence, following[:, None]], dim=1)
            out = _logits_of(model(sequence))
        return out[:, -1, :].float()


def _probe_tokens(model):
    """A short token sequence valid for this model's vocabulary, on the model's device."""
    import torch

    vocabulary = getattr(model, "vocab_size", None) or 32000
    device = next((b.device for b in model.buffers()), None) if hasattr(model, "buffers") else None
    if device is None:
        device = next((p.device for p in model.parameters()), torch.device("cpu"))
    return torch.tensor([[index % max(vocabulary - 1, 1) + 1 for index in range(8)]], device=device)


def _surfaces(model):
    """Names of the layer attributes that currently have replacements bound."""
    from .integrations.torch_lm import _model_layers

    watched = ("mlp", "self_attn", "linear_attn", "input_layernorm", "post_attention_layernorm")
    found = []
    for layer in _model_layers(model):
        for name in watched:
            member = getattr(layer, name, None)
            if member is None or name in found:
                continue
            implementation = getattr(type(member), "forward", None)
            if getattr(implementation, "_metile_original", None) is not None:
                found.append(name)
        block = getattr(type(layer), "forward", None)
        if getattr(block, "_metile_original", None) is not None and "block" not in found:
            found.append("block")
    return tuple(found)


@dataclass
class _Outcome:
    """One candidate feature set applied to the model: the live patch handle when it was accepted."""

    selected: tuple
    handle: object = None
    difference: float | None = None
    ran: bool = True

    @property
    def accepted(self):
        return self.handle is not None

    def release(self):
        if self.handle is not None:
            self.handle.__exit__(None, None, None)
            self.handle = None


class _Verifier:
    """Applies feature sets to one model and judges each against the unpatched logits.

    The unpatched logits are taken once, at construction.  When the model cannot even run unpatched,
    verification is switched off and the reason is kept for the report (the reference does the same,
    metile/compile.py:168-178)."""

    def __init__(self, model, verify, tolerance):
        self.model = model
        self.tolerance = tolerance
        self.enabled = bool(verify)
        self.failure = None
        self.tokens = None
        self.reference = None
        self.magnitude = 1.0
        if self.enabled:
            try:
                self.tokens = _probe_tokens(model)
                self.reference = _decode_logits(model, self.tokens)
                self.magnitude = max(float(self.reference.abs().max().item()), 1e-9)
            except Exception as error:
                self.failure = f"could not run the model unpatched ({type(error).__name__})"
                self.enabled = False

    def _distance(self):
        return float((_decode_logits(self.model, self.tokens) - self.reference).abs().max().item())

    def apply(self, selected):
        """Patch the model with exactly `selected`; keep the patch only if the logits agree."""
        from .integrations.torch_lm import apply_metile_to_torch_lm

        selected = tuple(selected)
        handle = apply_metile_to_torch_lm(model=self.model, **{name: name in selected for name in FEATURES})
        handle.__enter__()
        outcome = _Outcome(selected=selected, handle=handle)
        if not self.enabled:
            return outcome
        try:
            outcome.difference = self._distance()
        except Exception:
            outcome.ran = False
            outcome.release()
            return outcome
        # `not (d <= bound)` rather than `d > bound`: a NaN distance must be rejected too.
        if not outcome.difference <= self.tolerance * self.magnitude:
            outcome.release()
        return outcome

    def explain(self, outcome):
        """Why a single feature was declined, in the report's wording."""
        if not outcome.ran or not outcome.difference:
            return "could not run"
        relative = outcome.difference / self.magnitude
        if relative <= REORDERING_SCALE:
            scale = "reduction-order scale, raise tolerance to keep it"
        else:
            scale = "far beyond rounding, so a different computation"
        return f"changed the logits by {outcome.difference:g}, {relative:.1e} relative -- {scale}"


def _largest_verified_set(verifier, requested, declined):
    """The whole set if it verifies; otherwise every feature is judged alone and the survivors are
    re-applied together (dropping the last one while the combination still disagrees)."""
    outcome = verifier.apply(requested)
    if outcome.accepted or not verifier.enabled:
        return outcome
    declined["combined"] = "the full feature set changed the logits; bisected"
    survivors = []
    for feature in requested:
        alone = verifier.apply((feature,))
        if alone.accepted:
            alone.release()
            survivors.append(feature)
        else:
            declined[feature] = verifier.explain(alone)
    while survivors:
        outcome = verifier.apply(survivors)
        if outcome.accepted:
            return outcome
        survivors.pop()
    return _Outcome(selected=())


def compile(model, *, verify=True, features=FEATURES, tolerance=TOLERANCE):
    """Accelerate a torch model in place and report what changed.

    Returns a `CompileReport`, falsy when nothing was replaced; `.restore()` puts the model's own
    implementations back.  `tolerance` is relative to the largest reference logit and defaults to
    exact; raising it to about 5e-3 admits differences at the scale of a summation reorder, and the
    report names every feature it declined and by how much."""
    if model is None or not callable(model):
        raise TypeError("compile expects a loaded model")

    name = type(getattr(model, "model", model)).__name__
    requested = tuple(feature for feature in FEATURES if feature in features)
    declined = {}
    verifier = _Verifier(model, verify, tolerance)
    if verifier.failure:
        declined["verification"] = verifier.failure

    outcome = _largest_verified_set(verifier, requested, declined)
    if not outcome.accepted:
        return CompileReport(model=name, verified=False if verifier.enabled else None, declined=declined)

    surfaces = _surfaces(model)
    if not surfaces:
        outcome.release()
        declined["surfaces"] = "no layer in this model uses a class that can be replaced"
        return CompileReport(model=name, verified=None, declined=declined)

    # Per-call refusals recorded while the patched model ran: the original forward served those
    # calls; nothing was rerouted to another kernel.
    refusals = getattr(outcome.handle, "refusals", {})
    for surface, reason in refusals.items():
        declined.setdefault(surface, f"refused at call time -- {reason}")
    measured = verifier.enabled and outcome.difference is not None
    return CompileReport(
        model=name,
        features=tuple(feature for feature in outcome.selected if feature not in refusals),
        surfaces=surfaces,
        verified=True if verifier.enabled else None,
        difference=outcome.difference,
        relative=(outcome.difference / verifier.magnitude) if measured else None,
        declined=declined,
        handle=outcome.handle,
    )
