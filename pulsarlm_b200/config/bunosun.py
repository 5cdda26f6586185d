"""BunosunConfig: the typed configuration of the Bunosun decoder.

Bunosun lists its layers one by one. A layer's two sublayers read the same residual
stream, each through a norm of its own (weights stored around zero), and their outputs
enter it together, each scaled per channel. The mixer is differential attention over a
sliding window (two softmax maps per head over one set of values, rotary positions on
neighbouring pairs with linear scaling) or a gated delta rule with a decay per key
channel and short convolutions on q, k and v; the feed-forward is a mixture of experts
with grouped routing and a shared expert, or absent. A run of layers may be repeated
with the same weights (`loop`), every pass with a cache and state of its own and the
embedding's output added to the stream again before every pass but the first.
"""

from __future__ import annotations

import dataclasses

from .base import ConfigError, read_field, require_positive

MIXERS = ("attention", "channel_delta")


@dataclasses.dataclass(frozen=True)
class BunosunExperts:
    """A layer's `mlp` of kind "moe"."""

    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int | None = None   # None: no shared expert


@dataclasses.dataclass(frozen=True)
class BunosunLayer:
    """One entry of config.json's `layers`. Fields a mixer kind does not have are None."""

    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    mlp: BunosunExperts | None
    # attention
    diff: float | None = None
    scale: float | None = None
    window: int | None = None          # None: every earlier token
    rot_dims: int = 0                  # 0: no rotation
    rot_base: float = 10000.0
    rot_factor: float = 1.0
    # channel_delta
    taps: int | None = None
    decay_rank: int | None = None      # inner sizes of the decay's and the gate's projections: None takes
    gate_rank: int | None = None       # them from the stored tensors' shapes (random weights need them named)


@dataclasses.dataclass(frozen=True)
class BunosunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[BunosunLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    def runs(self) -> tuple[list[int], list[int]]:
        """(the layers in the order they run, the places in that order where a pass after the
        first begins)."""
        body = list(range(self.loop_start, self.loop_stop))
        order = list(range(self.loop_start))
        again = []
        for time in range(self.loop_times if body else 0):
            if time > 0:
                again.append(len(order))
            order += body
        order += list(range(self.loop_stop if body else self.loop_start, len(self.layers)))
        return order, again

    @staticmethod
    def from_text(text: dict) -> "BunosunConfig":
        layers_text = read_field(text, "layers", list)
        if not layers_text:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers = []
        for i, entry in enumerate(layers_text):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = read_field(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is unknown (known: {', '.join(MIXERS)})")
            mixer = read_field(entry, "mixer", dict)
            heads = read_field(mixer, "heads", int)
            kv_heads = read_field(mixer, "kv_heads", int, heads)
            dim, vdim = read_field(mixer, "dim", int), read_field(mixer, "vdim", int)
            for name, value in (("heads", heads), ("kv_heads", kv_heads), ("dim", dim), ("vdim", vdim)):
                require_positive(f"{where}.mixer.{name}", value)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}.mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
            mlp = _read_mlp(entry.get("mlp"), where)
            if kind == "attention":
                mask = mixer.get("mask")
                window = read_field(mask, "size", int) if isinstance(mask, dict) else None
                if window is not None:
                    require_positive(f"{where}.mixer.mask.size", window)
                rot = mixer.get("rot") or {}
                rot_dims = read_field(rot, "dims", int, 0)
                if rot_dims % 2 or not 0 <= rot_dims <= dim:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {rot_dims} must be even and at most dim {dim}")
                scaling = rot.get("scaling") or {}
                layers.append(BunosunLayer(
                    kind, heads, kv_heads, dim, vdim, mlp, diff=read_field(mixer, "diff", float),
                    scale=read_field(mixer, "scale", float), window=window, rot_dims=rot_dims,
                    rot_base=read_field(rot, "base", float, 10000.0), rot_factor=read_field(scaling, "factor", float, 1.0)))
            else:
                taps = read_field(mixer, "conv", int)
                require_positive(f"{where}.mixer.conv", taps)
                layers.append(BunosunLayer(kind, heads, kv_heads, dim, vdim, mlp, taps=taps,
                                           decay_rank=read_field(mixer, "decay_rank", int, None),
                                           gate_rank=read_field(mixer, "gate_rank", int, None)))
        loop = text.get("loop") or {}
        start, stop = read_field(loop, "start", int, 0), read_field(loop, "stop", int, 0)
        times = read_field(loop, "times", int, 1)
        if not 0 <= start <= stop <= len(layers) or times < 1:
            raise ConfigError(f"config.json: loop start {start}, stop {stop}, times {times} do not fit {len(layers)} layers")
        norm = read_field(text, "norm", dict)
        embedding = text.get("embedding") or {}
        cfg = BunosunConfig(
            architecture=str(text.get("architecture") or "Bunosun"),
            vocab=read_field(text, "vocab", int),
            width=read_field(text, "width", int),
            norm_eps=read_field(norm, "eps", float),
            embedding_scale=read_field(embedding, "scale", float, 1.0),
            layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times,
        )
        require_positive("vocab", cfg.vocab)
        require_positive("width", cfg.width)
        return cfg

    def to_text(self) -> dict:
        """A config.json that `from_text` reads back to an equal configuration."""
        layers = []
        for layer in self.layers:
            mixer: dict = {"heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim, "vdim": layer.vdim}
            if layer.type == "attention":
                mixer.update(diff=layer.diff, scale=layer.scale)
                if layer.window is not None:
                    mixer["mask"] = {"size": layer.window}
                if layer.rot_dims:
                    mixer["rot"] = {"base": layer.rot_base, "dims": layer.rot_dims,
                                    "scaling": {"factor": layer.rot_factor}}
            else:
                mixer["conv"] = layer.taps
                if layer.decay_rank is not None:
                    mixer["decay_rank"] = layer.decay_rank
                if layer.gate_rank is not None:
                    mixer["gate_rank"] = layer.gate_rank
            mlp = None
            if layer.mlp is not None:
                m = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": m.ff},
                       "router": {"experts": m.experts, "top": m.top, "groups": {"count": m.groups, "keep": m.keep}}}
                if m.shared_ff is not None:
                    mlp["shared"] = {"ff": m.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}


def _read_mlp(mlp, where: str) -> BunosunExperts | None:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be an object or null")
    kind = read_field(mlp, "kind", str, "moe")
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.mlp.kind {kind!r} is unsupported (supported: 'moe')")
    router = read_field(mlp, "router", dict)
    groups = router.get("groups") or {}
    shared = mlp.get("shared")
    out = BunosunExperts(
        experts=read_field(router, "experts", int), top=read_field(router, "top", int),
        ff=read_field(read_field(mlp, "expert", dict), "ff", int),
        groups=read_field(groups, "count", int, 1), keep=read_field(groups, "keep", int, read_field(groups, "count", int, 1)),
        shared_ff=read_field(shared, "ff", int) if isinstance(shared, dict) else None)
    for name, value in (("router.experts", out.experts), ("router.top", out.top), ("expert.ff", out.ff),
                        ("router.groups.count", out.groups), ("router.groups.keep", out.keep)):
        require_positive(f"{where}.mlp.{name}", value)
    if out.experts % out.groups or out.keep > out.groups or out.top > out.keep * (out.experts // out.groups):
        raise ConfigError(f"config.json: {where}.mlp.router: {out.top} of {out.experts} experts in {out.groups} groups "
                          f"of which {out.keep} stay cannot be chosen")
    return out
