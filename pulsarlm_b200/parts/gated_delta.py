"""The gated delta rule with a decay per key channel: a recurrent mixer with a matrix state
per head, its q, k and v filtered by a short convolution over time."""

from __future__ import annotations

import torch

from ..kernels import ops
from .delta_rule import SEQUENCE_ROWS_KEY, sequence_rows_plan
from .linear import linear
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, StateNeed, TensorNeed


@register_part("mixer", "channel_delta")
class ChannelDelta(Part):
    """Per head a state S [dim, vdim] (key channel x value channel), fp32, carried from token
    to token:

        q, k = silu(conv(Wq h)), silu(conv(Wk h))     [qk_heads, dim];   v = silu(conv(Wv h))  [heads, vdim]
        q^ = q / sqrt(|q|^2 + unit_eps) * dim^(-1/2);  k^ = k / sqrt(|k|^2 + unit_eps)
        b = sigmoid(Wb h)                                               one per head
        g = exp(-exp(A_log) * softplus(Wa2 (Wa1 h) + dt_bias))           per head and key channel
        S <- diag(g) S;  u = b * (v - S^T k^);  S <- S + k^ u^T;  o = S^T q^
        out = Wo (o / sqrt(mean(o^2) + eps) * norm * sigmoid(Wg2 (Wg1 h)))

    Head h reads q/k head h // (heads / qk_heads). The convolutions are causal, per channel,
    without bias (weight [channels, taps], the last tap the current token's); their last
    taps - 1 inputs are state too. Everything that reads h runs as one product (q, k, v, b
    and the inner projections of the decay and the gate stacked into one operand); the three
    convolutions are one kernel over the stacked channels; the recurrence is one kernel in
    fp32 (csrc/gated_delta.cu).

    params: hidden_size, n_heads, qk_heads, head_dim, value_dim, taps, eps (of the per-head
    norm), unit_eps (default 1e-6). tensors: q, k [qk*hd, H], v [nh*vd, H], q_conv, k_conv,
    v_conv [channels, taps], b [nh, H], a1 [ra, H], a2 [nh*hd, ra], g1 [rg, H], g2 [nh*vd, rg]
    (ra, rg: whatever the checkpoint holds unless `decay_rank` / `gate_rank` name them),
    A_log [nh], dt_bias [nh*hd], norm [vd], o [H, nh*vd]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.qk_heads = int(p.get("qk_heads") or self.n_heads)
        self.dim = int(self.param("head_dim"))
        self.vdim = int(self.param("value_dim"))
        self.taps = int(self.param("taps"))
        self.eps = float(self.param("eps"))
        self.unit_eps = float(p["unit_eps"]) if p.get("unit_eps") is not None else 1e-6
        if self.n_heads % self.qk_heads:
            raise ValueError(f"channel_delta: {self.n_heads} heads are not a multiple of {self.qk_heads} q/k heads")
        if self.taps < 1:
            raise ValueError(f"channel_delta: taps must be at least 1, got {self.taps}")
        self.channels = 2 * self.qk_heads * self.dim + self.n_heads * self.vdim
        self.stacked = self.conv = self.a2 = self.g2 = self.o = None
        self.a_log = self.dt_bias = self.norm = None
        self.rank_a = self.rank_g = 0
        self.states = None
        self.filter_state = FilterState(self.taps, self.channels)

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, hd, vd, taps = (int(p[k]) for k in ("hidden_size", "n_heads", "head_dim", "value_dim", "taps"))
        qk = int(p.get("qk_heads") or nh)
        ra = int(p["decay_rank"]) if p.get("decay_rank") is not None else -1
        rg = int(p["gate_rank"]) if p.get("gate_rank") is not None else -1
        return {
            t["q"]: TensorNeed((qk * hd, h)), t["k"]: TensorNeed((qk * hd, h)), t["v"]: TensorNeed((nh * vd, h)),
            t["q_conv"]: TensorNeed((qk * hd, taps)), t["k_conv"]: TensorNeed((qk * hd, taps)),
            t["v_conv"]: TensorNeed((nh * vd, taps)),
            t["b"]: TensorNeed((nh, h)),
            t["a1"]: TensorNeed((ra, h)), t["a2"]: TensorNeed((nh * hd, ra)),
            t["g1"]: TensorNeed((rg, h)), t["g2"]: TensorNeed((nh * vd, rg)),
            t["A_log"]: TensorNeed((nh,), role="offset"), t["dt_bias"]: TensorNeed((nh * hd,), role="offset"),
            t["norm"]: TensorNeed((vd,), role="vector"), t["o"]: TensorNeed((h, nh * vd)),
        }

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.rank_a, self.rank_g = int(tensors[t["a1"]].shape[0]), int(tensors[t["g1"]].shape[0])
        if tensors[t["a2"]].shape[1] != self.rank_a or tensors[t["g2"]].shape[1] != self.rank_g:
            raise ValueError("channel_delta: the inner and outer projections of the decay or the gate disagree")
        # One operand for everything that reads h: the filtered channels first (their rows start
        # the product's output, so the convolution reads them in place), then b, a1, g1.
        self.stacked = torch.cat([tensors[t[n]] for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
        self.conv = torch.cat([tensors[t[n]].float() for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a2 = tensors[t["a2"]].contiguous()
        self.g2 = tensors[t["g2"]].contiguous()
        self.o = tensors[t["o"]].contiguous()
        self.a_log = tensors[t["A_log"]].float().contiguous()
        self.dt_bias = tensors[t["dt_bias"]].float().contiguous()
        self.norm = tensors[t["norm"]].float().contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.dim, self.vdim), dtype="float32")

    def bind_cache(self, binding) -> None:
        self.states = binding.states

    def state_holders(self) -> list:
        """What else keeps something per request for this mixer: the convolutions' inputs."""
        return [self.filter_state]

    def captures_state_steps(self) -> bool:
        return True

    def plan_key(self):
        return SEQUENCE_ROWS_KEY

    def plan_step(self, step) -> dict:
        return sequence_rows_plan(step)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, qk, hd, vd, c = self.n_heads, self.qk_heads, self.dim, self.vdim, self.channels
        proj = linear(h, self.stacked)                       # [T, c + nh + ra + rg]
        filtered = torch.empty((tokens, c), dtype=h.dtype, device=h.device)
        conv_states = self.filter_state.states(h)
        # (a step of single tokens: the convolution and its state's update in one launch)
        single = self.taps > 1 and int(batch.n_decode) == tokens
        if not (single and ops.short_conv_single(proj[:, :c], self.conv, conv_states, batch.entry, batch.slots,
                                                 filtered, residual=False, act="silu")):
            ops.short_conv_act(proj[:, :c], self.conv, conv_states, batch.entry, batch.slots, filtered,
                               residual=False, act="silu")
            if self.taps > 1:
                ops.short_conv_state_strided(proj[:, :c], batch.entry, batch.slots, conv_states)
        b_pre = proj[:, c:c + nh]
        a_pre = linear(proj[:, c + nh:c + nh + self.rank_a], self.a2)
        gate_pre = linear(proj[:, c + nh + self.rank_a:], self.g2)
        plan = batch.plans[SEQUENCE_ROWS_KEY]
        out = torch.empty((tokens, nh * vd), dtype=h.dtype, device=h.device)
        ops.gated_delta(filtered[:, :qk * hd], filtered[:, qk * hd:2 * qk * hd], filtered[:, 2 * qk * hd:], b_pre,
                        a_pre, gate_pre, self.a_log, self.dt_bias, self.norm, self.states, plan["first"],
                        plan["count"], batch.slots, out, nh, qk, hd, vd, self.unit_eps, hd ** -0.5, self.eps)
        return linear(out, self.o)


class FilterState:
    """The last taps - 1 inputs of a mixer's convolutions, per request: [taps - 1, channels] in
    the engine's dtype (what the projection wrote, so a cut changes no bit). A cache holder
    beside the mixer that owns it."""

    def __init__(self, taps: int, channels: int):
        self.taps, self.channels = taps, channels
        self.binding = None

    def cache_need(self) -> StateNeed | None:
        return StateNeed((self.taps - 1, self.channels), dtype="engine") if self.taps > 1 else None

    def bind_cache(self, binding) -> None:
        self.binding = binding

    def captures_state_steps(self) -> bool:
        return True

    def states(self, like: torch.Tensor) -> torch.Tensor:
        if self.taps == 1:
            return torch.empty((1, 0, self.channels), dtype=like.dtype, device=like.device)
        return self.binding.states
