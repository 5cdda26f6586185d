"""A short causal convolution over time in front of a sublayer's input."""

from __future__ import annotations

import os

import torch

from ..kernels import ops
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, StateNeed, TensorNeed


FUSE_DECODE = os.environ.get("PULSARLM_B200_FUSE_CONV", "1") != "0"  # (0: always the separate kernels, for comparison)


@register_part("filter", "short_conv")
class ShortConv(Part):
    """h <- h + conv(h): per channel, conv(h)[t] = sum_j w[:, j] * h[t - (taps - 1) + j]
    over the sequence's own earlier inputs, zeros before its start. The last taps - 1
    inputs are the sequence's state between steps (a slot per request, in the engine's
    dtype). params: hidden_size, taps. tensors: weight [hidden_size, taps] (kept fp32)."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.taps = int(self.param("taps"))
        if self.taps < 1:
            raise ValueError(f"short_conv: taps must be at least 1, got {self.taps}")
        self.weight: torch.Tensor | None = None
        self.binding = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        return {spec.tensors["weight"]: TensorNeed((int(spec.params["hidden_size"]), int(spec.params["taps"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].float().contiguous()

    def cache_need(self) -> StateNeed | None:
        if self.taps == 1:
            return None
        return StateNeed((self.taps - 1, self.hidden), dtype="engine")

    def bind_cache(self, binding) -> None:
        self.binding = binding

    def captures_state_steps(self) -> bool:
        return True  # (no host round trip: the state moves on inside the step's kernels)

    def rides_along(self, batch) -> tuple | None:
        """In a step whose entries bring one token each, what the norm kernel in front needs to
        do this part's work too (see ops.add_normed_rmsnorm): one launch instead of three."""
        if not FUSE_DECODE or int(batch.n_decode) != int(batch.n_tokens):
            return None
        if self.taps == 1:
            return (self.weight, torch.empty((1, 0, self.hidden), dtype=self.ctx.dtype, device=self.weight.device),
                    batch.slots)
        return (self.weight, self.binding.states, batch.slots)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        out = torch.empty_like(h)
        if self.taps == 1:
            state = torch.empty((1, 0, self.hidden), dtype=h.dtype, device=h.device)
            ops.short_conv(h, self.weight, state, batch.entry, batch.slots, out)
            return out
        states = self.binding.states
        ops.short_conv(h, self.weight, states, batch.entry, batch.slots, out)
        ops.short_conv_state(h, batch.entry, batch.slots, states)
        return out
