"""RerilornConfig: the typed configuration of the Rerilorn decoder.

Rerilorn lists its layers one by one; each has a mixer of one of two kinds (a
generalized-delta-rule recurrence, or attention over a cached low-rank latent with a
sliding window and a sink), an optional dense feed-forward, norms before and after
every sublayer and a short convolution over time in front of every sublayer's input.
"""

from __future__ import annotations

import dataclasses

from .base import ConfigError, read_field, require_positive

MIXERS = ("general_delta", "latent_attention")


@dataclasses.dataclass(frozen=True)
class RerilornLayer:
    """One entry of config.json's `layers`. Fields a mixer kind does not have are None."""

    type: str
    heads: int
    dim: int
    ff: int | None                 # None: the layer has no feed-forward
    value_dim: int | None = None   # latent_attention
    latent_rank: int | None = None
    window: int | None = None      # None: every earlier token
    scale: float | None = None
    decay_rank: int | None = None  # general_delta: None takes it from the stored tensors' shapes


@dataclasses.dataclass(frozen=True)
class RerilornConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    taps: int                      # 0: no convolution in front of the sublayers
    layers: tuple[RerilornLayer, ...]

    @staticmethod
    def from_text(text: dict) -> "RerilornConfig":
        layers_text = read_field(text, "layers", list)
        if not layers_text:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers = []
        for i, entry in enumerate(layers_text):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_field(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown (known: {', '.join(MIXERS)})")
            mixer = read_field(entry, "mixer", dict)
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
                mlp_kind = read_field(mlp, "kind", str, "dense")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp_kind!r} is unsupported (supported: "
                                      f"'dense')")
                ff = read_field(mlp, "ff", int)
                require_positive(f"layers[{i}].mlp.ff", ff)
            heads, dim = read_field(mixer, "heads", int), read_field(mixer, "dim", int)
            require_positive(f"layers[{i}].mixer.heads", heads)
            require_positive(f"layers[{i}].mixer.dim", dim)
            if kind == "general_delta":
                layers.append(RerilornLayer(kind, heads, dim, ff, decay_rank=read_field(mixer, "decay_rank", int, None)))
            else:
                mask = mixer.get("mask")
                window = read_field(mask, "size", int) if isinstance(mask, dict) else None
                if window is not None:
                    require_positive(f"layers[{i}].mixer.mask.size", window)
                rank, vdim = read_field(mixer, "kv_rank", int), read_field(mixer, "vdim", int)
                require_positive(f"layers[{i}].mixer.kv_rank", rank)
                require_positive(f"layers[{i}].mixer.vdim", vdim)
                layers.append(RerilornLayer(kind, heads, dim, ff, value_dim=vdim, latent_rank=rank, window=window,
                                            scale=read_field(mixer, "scale", float)))
        norm = read_field(text, "norm", dict)
        canon = text.get("canon") or {}
        embedding = text.get("embedding") or {}
        cfg = RerilornConfig(
            architecture=str(text.get("architecture") or "Rerilorn"),
            vocab=read_field(text, "vocab", int),
            width=read_field(text, "width", int),
            norm_eps=read_field(norm, "eps", float),
            residual_mult=read_field(text, "residual_mult", float, 1.0),
            embedding_scale=read_field(embedding, "scale", float, 1.0),
            taps=read_field(canon, "taps", int, 0),
            layers=tuple(layers),
        )
        require_positive("vocab", cfg.vocab)
        require_positive("width", cfg.width)
        if cfg.taps < 0:
            raise ConfigError(f"config.json: canon.taps must not be negative, got {cfg.taps}")
        return cfg

    def to_text(self) -> dict:
        """A config.json that `from_text` reads back to an equal configuration."""
        layers = []
        for layer in self.layers:
            if layer.type == "general_delta":
                mixer = {"heads": layer.heads, "dim": layer.dim}
                if layer.decay_rank is not None:
                    mixer["decay_rank"] = layer.decay_rank
            else:
                mixer = {"heads": layer.heads, "dim": layer.dim, "vdim": layer.value_dim, "kv_rank": layer.latent_rank,
                         "scale": layer.scale}
                if layer.window is not None:
                    mixer["mask"] = {"size": layer.window}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        text = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.taps:
            text["canon"] = {"taps": self.taps}
        return text
