"""Arrangements of norms, mixer and feed-forward around the residual stream.

A block's forward takes the fp32 residual stream `x` and the previous block's
not-yet-added output `delta`, and returns the same pair: the add is done inside
the next norm kernel (one pass over x instead of two).
"""

from __future__ import annotations

import torch

from . import native_layer
from .basic import NormedDelta
from .registry import BuildContext, build_part, register_part
from .spec import LayerSpec


@register_part("block", "pre_norm")
class PreNormBlock:
    """x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x))
    (pulsarlm-core/src/engine/model/llama.cpp:88-92). Norm names in the
    LayerSpec: "mixer" and "feed_forward"."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
        self._native: bool | None = None  # whether the parts are the ones the native layer call takes

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        """(kind, PartSpec) of every part, so tensor needs can be listed without building."""
        return [("norm", spec.norms["mixer"]), ("mixer", spec.mixer),
                ("norm", spec.norms["feed_forward"]), ("feed_forward", spec.feed_forward)]

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, batch) -> tuple[torch.Tensor, torch.Tensor]:
        # The standard parts in bfloat16: the whole layer from one native call (the same kernels
        # in the same order; see native_layer.py). Anything else: the parts' own calls below.
        if self._native is None:
            self._native = native_layer.eligible(self)
        if self._native:
            done = native_layer.forward(self, x, delta, batch)
            if done is not None:
                return done
        h = self.mixer_norm.forward(x, delta)
        mixed = self.mixer.forward(h, batch)
        h = self.ff_norm.forward(x, mixed)
        return x, self.feed_forward.forward(h, batch)


@register_part("block", "sandwich_norm")
class SandwichNormBlock:
    """Every sublayer is normed before and after, and its normed output enters the
    residual stream scaled:

        x += m * norm_mixer_out(mixer(filter_mixer(norm_mixer(x))))
        x += m * norm_ff_out(feed_forward(filter_ff(norm_ff(x))))

    Norm names in the LayerSpec: "mixer", "mixer_out", "feed_forward", "feed_forward_out".
    `extras` of the LayerSpec: "residual_mult" (m, 1 when absent) and optional PartSpecs
    "mixer_filter" / "feed_forward_filter" of the "filter" registry (e.g. a short
    convolution over time), applied to the sublayer's input. A LayerSpec whose
    feed_forward is None has the first line only. The out-norm of a sublayer is not run
    on its own: its output travels as a NormedDelta and the next norm kernel norms it,
    adds it and norms the sum for the next sublayer in one pass."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        extras = spec.extras or {}
        self.mult = float(extras.get("residual_mult", 1.0))
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer_out_norm = build_part("norm", spec.norms["mixer_out"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.mixer_filter = build_part("filter", extras["mixer_filter"], ctx) if extras.get("mixer_filter") else None
        self.feed_forward = self.ff_norm = self.ff_out_norm = self.ff_filter = None
        if spec.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
            self.ff_out_norm = build_part("norm", spec.norms["feed_forward_out"], ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
            if extras.get("feed_forward_filter"):
                self.ff_filter = build_part("filter", extras["feed_forward_filter"], ctx)

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        extras = spec.extras or {}
        out = [("norm", spec.norms["mixer"]), ("norm", spec.norms["mixer_out"]), ("mixer", spec.mixer)]
        if extras.get("mixer_filter"):
            out.append(("filter", extras["mixer_filter"]))
        if spec.feed_forward is not None:
            out += [("norm", spec.norms["feed_forward"]), ("norm", spec.norms["feed_forward_out"]),
                    ("feed_forward", spec.feed_forward)]
            if extras.get("feed_forward_filter"):
                out.append(("filter", extras["feed_forward_filter"]))
        return out

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer_out_norm, self.mixer, self.mixer_filter, self.ff_norm,
                            self.ff_out_norm, self.feed_forward, self.ff_filter) if p is not None]

    def cache_holders(self):
        """The parts that keep something per request, the mixer first."""
        return [self.mixer] + [f for f in (self.mixer_filter, self.ff_filter) if f is not None]

    @staticmethod
    def _input(norm, filt, x, delta, batch):
        """A sublayer's input: the norm (with the pending output added first), then the filter.
        Where the filter can ride along in the norm's kernel (a step of single tokens), one launch."""
        if filt is None:
            return norm.forward(x, delta)
        ride = getattr(filt, "rides_along", None)
        conv = ride(batch) if ride is not None and isinstance(delta, NormedDelta) else None
        if conv is not None:
            return norm.forward(x, delta, conv=conv)
        return filt.forward(norm.forward(x, delta), batch)

    def forward(self, x: torch.Tensor, delta, batch):
        h = self._input(self.mixer_norm, self.mixer_filter, x, delta, batch)
        delta = self.mixer_out_norm.pending(self.mixer.forward(h, batch), self.mult)
        if self.feed_forward is None:
            return x, delta
        h = self._input(self.ff_norm, self.ff_filter, x, delta, batch)
        # A bias on the feed-forward's last projection is added by the kernel that norms its output.
        bias = getattr(self.feed_forward, "down_bias", None)
        if bias is not None:
            y = self.feed_forward.forward(h, batch, bias_taken=True)
        else:
            y = self.feed_forward.forward(h, batch)
        return x, self.ff_out_norm.pending(y, self.mult, bias)
