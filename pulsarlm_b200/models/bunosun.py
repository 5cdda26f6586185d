"""The Bunosun decoder, described as data and registered by name.

A layer: x += ls1 * mixer(norm1(x)) + ls2 * ff(norm2(x)), both sublayers reading the same
x (the "parallel" block; norm weights stored around zero). The embedding is scaled. A run
of layers may repeat with the same weights; every pass has a cache of its own and the
embedding's output joins the stream again before every pass but the first. Tensor names:
`embed`, `final.norm`, `head`, and per layer `l<i>.` + norm1, norm2, ls1, ls2, mix.*, mlp.*.
"""

from __future__ import annotations

from ..config.bunosun import BunosunConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def describe_bunosun(cfg: BunosunConfig) -> ModelSpec:
    width = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": width, "eps": cfg.norm_eps, "unit_offset": True}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        if layer.type == "attention":
            position = (PartSpec("rope_pairs", {"theta": layer.rot_base, "rotary_dim": layer.rot_dims,
                                                "factor": layer.rot_factor}) if layer.rot_dims
                        else PartSpec("none"))
            mixer = PartSpec(
                "diff_attention",
                {"hidden_size": width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                 "value_dim": layer.vdim, "diff": layer.diff, "scale": layer.scale, "window": layer.window,
                 "eps": cfg.norm_eps, "position": position},
                {name: m + name for name in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")})
        else:
            mixer = PartSpec(
                "channel_delta",
                {"hidden_size": width, "n_heads": layer.heads, "qk_heads": layer.kv_heads, "head_dim": layer.dim,
                 "value_dim": layer.vdim, "taps": layer.taps, "eps": cfg.norm_eps, "decay_rank": layer.decay_rank,
                 "gate_rank": layer.gate_rank},
                {**{name: m + name for name in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "A_log", "dt_bias", "norm",
                                                 "o")},
                 "q_conv": m + "q.conv", "k_conv": m + "k.conv", "v_conv": m + "v.conv"})
        norms = {"mixer": norm(p + "norm1")}
        extras = {"mixer_scale": p + "ls1"}
        feed_forward = None
        if layer.mlp is not None:
            e = layer.mlp
            f = p + "mlp."
            tensors = {"router": f + "router", "correction": f + "correction", "expert_gate": f + "e{e}.gate",
                       "expert_up": f + "e{e}.up", "expert_down": f + "e{e}.down"}
            if e.shared_ff is not None:
                tensors.update(shared_gate=f + "shared.gate", shared_up=f + "shared.up", shared_down=f + "shared.down")
            feed_forward = PartSpec(
                "moe", {"hidden_size": width, "expert_size": e.ff, "n_experts": e.experts, "top": e.top,
                        "groups": e.groups, "keep_groups": e.keep, "shared_size": e.shared_ff}, tensors)
            norms["feed_forward"] = norm(p + "norm2")
            extras["feed_forward_scale"] = p + "ls2"
        layers.append(LayerSpec(block="parallel", mixer=mixer, feed_forward=feed_forward, norms=norms, extras=extras))
    order, again = cfg.runs()
    sizes = {"vocab_size": cfg.vocab, "hidden_size": width}
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("table", {**sizes, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        layers=layers,
        order=order,
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(sizes), {"weight": "head"}),
        cache_per_run=True,
        rejoin_runs=tuple(again),
    )


register_architecture("Bunosun", BunosunConfig.from_text, describe_bunosun, model_types=("bunosun",), replace=True)
