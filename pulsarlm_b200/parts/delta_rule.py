"""The generalized-delta-rule mixer: a recurrent layer with a matrix state per head."""

from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from .linear import activated_linear, linear
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, StateNeed, TensorNeed


def sequence_rows_plan(step) -> dict:
    """What a kernel that walks each entry's rows in order needs on the device: the row of
    every entry's first token and how many rows it brings (int32 [entries] each)."""
    return {"first": np.asarray(step.first_rows, dtype=np.int32),
            "count": np.asarray(step.query_lens, dtype=np.int32)}


SEQUENCE_ROWS_KEY = ("sequence rows",)


@register_part("mixer", "general_delta")
class GeneralDelta(Part):
    """Per head a state S [dim, dim] (key channel x value channel), fp32, carried from
    token to token:

        r, k, v = Wr h, Wk h, Wv h                       (heads x dim each)
        w = exp(-decay_scale * sigmoid(Ww2 tanh(Ww1 h) + w0))      decay per key channel
        a = sigmoid(Wa h + a0)                                     removal rate per key channel
        u = k / sqrt(|k|^2 + unit_eps)                             per head
        S <- diag(w) S - (a * u) (u^T S) + k v^T ;  o = S^T r      (both products read the old S)
        out = Wo (rmsnorm_per_head(o) * norm * sigmoid(Wg h))

    The projections run as two matrix products (r, k, v, g, a and the decay's inner
    projection stacked into one operand; then the decay's outer projection); everything
    after them is one kernel in fp32 (csrc/delta_rule.cu).

    params: hidden_size, n_heads, head_dim, eps (of the per-head norm), decay_scale
    (default exp(-1/2)), unit_eps (default 1e-6). tensors: r, k, v, g, a [nh*hd, H],
    a_bias, w0, norm [nh*hd], w1 [L, H], w2 [nh*hd, L] (L = decay_rank, or whatever the
    checkpoint holds when that is None), o [H, nh*hd]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.eps = float(self.param("eps"))
        self.decay_scale = float(p["decay_scale"]) if p.get("decay_scale") is not None else math.exp(-0.5)
        self.unit_eps = float(p["unit_eps"]) if p.get("unit_eps") is not None else 1e-6
        # (None: the checkpoint's tensors give it)
        self.inner = int(p["decay_rank"]) if p.get("decay_rank") is not None else None
        self.stacked: torch.Tensor | None = None
        self.w2 = self.o = self.w0 = self.a0 = self.norm = None
        self.binding = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, width = int(p["hidden_size"]), int(p["n_heads"]) * int(p["head_dim"])
        inner = int(p["decay_rank"]) if p.get("decay_rank") is not None else -1
        needs = {t[name]: TensorNeed((width, h)) for name in ("r", "k", "v", "g", "a")}
        needs[t["w1"]] = TensorNeed((inner, h))
        needs[t["w2"]] = TensorNeed((width, inner))
        needs[t["o"]] = TensorNeed((h, width))
        needs[t["a_bias"]] = TensorNeed((width,), role="offset")
        needs[t["w0"]] = TensorNeed((width,), role="offset")
        needs[t["norm"]] = TensorNeed((width,), role="vector")
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        # One operand for everything that reads h; the decay's inner projection last.
        self.stacked = torch.cat([tensors[t[name]] for name in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.w2 = tensors[t["w2"]].contiguous()
        self.inner = int(tensors[t["w1"]].shape[0])
        if self.w2.shape[1] != self.inner:
            raise ValueError(f"general_delta: the decay's projections disagree: {t['w1']} has {self.inner} rows, "
                             f"{t['w2']} {self.w2.shape[1]} columns")
        self.o = tensors[t["o"]].contiguous()
        self.w0 = tensors[t["w0"]].float().contiguous()
        self.a0 = tensors[t["a_bias"]].float().contiguous()
        self.norm = tensors[t["norm"]].float().contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.head_dim, self.head_dim), dtype="float32")

    def bind_cache(self, binding) -> None:
        self.binding = binding

    def captures_state_steps(self) -> bool:
        return True

    def plan_key(self):
        return SEQUENCE_ROWS_KEY

    def plan_step(self, step) -> dict:
        return sequence_rows_plan(step)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        width = self.n_heads * self.head_dim
        proj = linear(h, self.stacked)                              # [T, 5 * width + inner]
        r, k, v, g, a = (proj[:, i * width:(i + 1) * width] for i in range(5))
        w_pre = activated_linear(proj[:, 5 * width:], None, "tanh", self.w2)   # the decay's inner activation
        plan = batch.plans[SEQUENCE_ROWS_KEY]
        out = torch.empty((tokens, width), dtype=h.dtype, device=h.device)
        ops.delta_rule(r, k, v, g, a, w_pre, self.w0, self.a0, self.norm, self.binding.states, plan["first"],
                       plan["count"], batch.slots, out, self.n_heads, self.head_dim, self.decay_scale, self.unit_eps,
                       self.eps)
        return linear(out, self.o)
