"""The Rerilorn decoder, described as data and registered by name.

A layer: x += m * norm1b(mixer(conv1(norm1(x)))), then, where the layer has a
feed-forward, x += m * norm2b(ff(conv2(norm2(x)))). The embedding is scaled; the head
is the embedding table itself, unscaled. Tensor names: `embed`, `final.norm`, and per
layer `l<i>.` + norm1, norm1b, norm2, norm2b, canon1, canon2, mix.*, mlp.*.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rerilorn import RerilornConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def describe_rerilorn(cfg: RerilornConfig) -> ModelSpec:
    width = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": width, "eps": cfg.norm_eps}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        if layer.type == "general_delta":
            mixer = PartSpec(
                "general_delta",
                {"hidden_size": width, "n_heads": layer.heads, "head_dim": layer.dim, "eps": cfg.norm_eps,
                 "decay_rank": layer.decay_rank},
                {"r": m + "r", "k": m + "k", "v": m + "v", "g": m + "g", "a": m + "a", "a_bias": m + "a.b",
                 "w1": m + "w1", "w2": m + "w2", "w0": m + "w0", "norm": m + "norm", "o": m + "o"})
        else:
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": width, "n_heads": layer.heads, "head_dim": layer.dim, "value_dim": layer.value_dim,
                 "latent_rank": layer.latent_rank, "scale": layer.scale, "window": layer.window, "eps": cfg.norm_eps,
                 "sink": True, "gate": True},
                {"q": m + "q", "down": m + "dkv", "latent_norm": m + "dkv.norm", "up_k": m + "uk", "up_v": m + "uv",
                 "sink": m + "sink", "gate": m + "g", "o": m + "o"})
        norms = {"mixer": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
        extras: dict = {"residual_mult": cfg.residual_mult}
        if cfg.taps:
            extras["mixer_filter"] = PartSpec("short_conv", {"hidden_size": width, "taps": cfg.taps},
                                              {"weight": p + "canon1"})
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec(
                "mlp", {"hidden_size": width, "intermediate_size": layer.ff, "activation": "relu2", "bias": True},
                {"up": p + "mlp.up", "up_bias": p + "mlp.up.b", "down": p + "mlp.down", "down_bias": p + "mlp.down.b"})
            norms["feed_forward"] = norm(p + "norm2")
            norms["feed_forward_out"] = norm(p + "norm2b")
            if cfg.taps:
                extras["feed_forward_filter"] = PartSpec("short_conv", {"hidden_size": width, "taps": cfg.taps},
                                                         {"weight": p + "canon2"})
        layers.append(LayerSpec(block="sandwich_norm", mixer=mixer, feed_forward=feed_forward, norms=norms,
                                extras=extras))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": width}
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("table", {**sizes, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        layers=layers,
        order=list(range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(sizes), {"weight": None}),
    )


register_architecture("Rerilorn", RerilornConfig.from_text, describe_rerilorn, model_types=("rerilorn",), replace=True)
