"""Small Bunosun configurations and random weights for the tests.

The configurations differ from each other in every size and constant: layer order, the
loop (absent, in the middle, from the start), widths, head counts (query heads per kv
head 1, 2 and 3), map, value and state sizes (value size equal to, above and below twice
the map size), windows (one layer without), rotary widths (none, part, all of a map) and
scaling, taps, experts, groups (one group; fewer kept than there are), a layer without
feed-forward, a feed-forward without shared expert. Weights are drawn with torch and
written with the `safetensors` package, so the engine's reader and its names are checked
against an independent file.
"""

from __future__ import annotations

import json
import os
import tempfile

import torch

import plain_bunosun


def moe(experts, top, ff, groups=1, keep=None, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep or groups}}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def attention_layer(heads, kv_heads, dim, vdim, window, rot_dims, mlp, diff=0.3, scale=None, base=10000.0, factor=1.0):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
             "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims, "scaling": {"factor": factor}}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def delta_layer(heads, kv_heads, dim, vdim, taps, mlp):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": taps}, "mlp": mlp}


CONFIG_A = {
    "architecture": "Bunosun", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [attention_layer(4, 2, 16, 32, 21, 8, moe(8, 2, 40, 4, 2, 56), diff=0.3, factor=2.0),
               delta_layer(4, 2, 16, 24, 3, moe(8, 2, 40, 4, 2, 56)),
               attention_layer(4, 2, 16, 32, 21, 8, moe(8, 2, 40, 4, 2, 56), diff=0.3, factor=2.0),
               delta_layer(2, 2, 16, 24, 3, None)],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
CONFIG_B = {
    "architecture": "Bunosun", "vocab": 97, "width": 40, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [delta_layer(2, 2, 24, 8, 4, None),
               attention_layer(2, 1, 12, 40, None, 12, moe(6, 1, 24), diff=0.6, scale=0.4, base=100.0),
               attention_layer(3, 3, 8, 8, 9, 0, moe(6, 1, 24), diff=0.1, scale=0.3)],
}
CONFIG_C = {
    "architecture": "Bunosun", "vocab": 128, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
    "layers": [attention_layer(3, 1, 32, 64, 40, 16, moe(12, 3, 48, 3, 2, 32), diff=0.5, scale=0.2, factor=4.0),
               delta_layer(2, 1, 64, 32, 2, moe(12, 3, 48, 3, 2, 32))],
    "loop": {"start": 0, "stop": 2, "times": 3},
}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 32), "C": (CONFIG_C, 16)}
INNER_RANK = 6


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,), "head": (cfg["vocab"], w)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "ls1"] = (w,)
        heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            shapes[p + "mix.q"] = (heads * 2 * dim, w)
            shapes[p + "mix.k"] = (kv * 2 * dim, w)
            shapes[p + "mix.v"] = (kv * vdim, w)
            for name in ("lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + name] = (dim,)
            shapes[p + "mix.o"] = (w, heads * vdim)
        else:
            taps = m["conv"]
            for name, rows in (("q", kv * dim), ("k", kv * dim), ("v", heads * vdim)):
                shapes[p + "mix." + name] = (rows, w)
                shapes[p + "mix." + name + ".conv"] = (rows, taps)
            shapes[p + "mix.b"] = (heads, w)
            shapes[p + "mix.A_log"] = (heads,)
            shapes[p + "mix.norm"] = (vdim,)
            shapes[p + "mix.a1"], shapes[p + "mix.a2"] = (INNER_RANK, w), (heads * dim, INNER_RANK)
            shapes[p + "mix.dt_bias"] = (heads * dim,)
            shapes[p + "mix.g1"], shapes[p + "mix.g2"] = (INNER_RANK, w), (heads * vdim, INNER_RANK)
            shapes[p + "mix.o"] = (w, heads * vdim)
        mlp = layer["mlp"]
        if mlp is not None:
            shapes[p + "norm2"] = shapes[p + "ls2"] = (w,)
            experts, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            shapes[p + "mlp.router"], shapes[p + "mlp.correction"] = (experts, w), (experts,)
            names = [f"e{e}" for e in range(experts)]
            sizes = {name: ff for name in names}
            if mlp.get("shared"):
                sizes["shared"] = mlp["shared"]["ff"]
            for name, size in sizes.items():
                shapes[f"{p}mlp.{name}.gate"] = shapes[f"{p}mlp.{name}.up"] = (size, w)
                shapes[f"{p}mlp.{name}.down"] = (w, size)
    return shapes


def random_weights(cfg: dict, seed: int, dtype: torch.dtype = torch.float32) -> dict:
    """Matrices N(0, 1/sqrt(in)) (queries and keys twice that, routers four times, so that
    attention and routing are far from uniform), norm weights 0.1 N around zero, layer scales
    0.5 + 0.1 N, the router's correction N(0, 0.1) (larger than most scores: choice scores go
    negative), convolution taps N(0, 0.5), the rest N(0, 0.5); rounded to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and "." in name else name
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * torch.randn(shape, generator=gen)
        elif leaf in ("ls1", "ls2"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=gen)
        elif leaf == "mix.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif leaf == "mlp.correction":
            t = 0.1 * torch.randn(shape, generator=gen)
        elif leaf.endswith(".conv"):
            t = 0.5 * torch.randn(shape, generator=gen)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen) / (cfg.get("embedding") or {}).get("scale", 1.0)
        else:
            gain = 4.0 if leaf == "mlp.router" else 2.0 if leaf in ("mix.q", "mix.k") else 1.0
            t = torch.randn(shape, generator=gen) * (gain / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def write_model_dir(folder: str, cfg: dict, weights: dict) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_tokens(cfg: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=gen).tolist()


# Largest |difference| over largest |expected| of a row of logits, against the plain implementation in
# float64. The float32 engine is the sharp comparison. In bfloat16 the engine rounds activations at
# some ten places a layer, and a routed layer can send a token whose two best choice scores are
# closer than a rounding to another expert, so the bfloat16 runs hold most positions to the bar and
# none beyond a loose one; what is off by a rounding is left to the float32 runs.
TOLERANCE = {"float32": 2e-4, "bfloat16": 6e-2}


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max())


class TinyBunosun:
    """A configuration with random weights rounded to the engine's dtype (so that the plain
    implementation, which runs in float64, and the engine start from identical numbers), its
    model folder, and the plain implementation's logits on demand."""

    def __init__(self, key: str, dtype: str, seed: int = 1, cfg: dict | None = None, weights: dict | None = None,
                 page: int = 16):
        self.cfg, self.page = CONFIGS[key] if cfg is None else (cfg, page)
        self.dtype = dtype
        torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.weights = weights if weights is not None else random_weights(self.cfg, seed, torch_dtype)
        self.plain_weights = {k: v.double() for k, v in self.weights.items()}
        self._dir = tempfile.TemporaryDirectory()
        self.folder = write_model_dir(self._dir.name, self.cfg, self.weights)
        self._plain: dict[tuple, torch.Tensor] = {}

    def plain_logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._plain:
            self._plain[key] = plain_bunosun.forward(self.cfg, self.plain_weights, list(tokens))[0]
        return self._plain[key]

    def runner(self, n_pages: int, slots: int = 4, page: int | None = None):
        from pulsarlm_b200.cache.manager import CacheManager
        from pulsarlm_b200.engine.loading import load_model
        from pulsarlm_b200.engine.runner import ModelRunner

        model = load_model(self.folder, self.dtype, "cuda:0")
        cache = CacheManager(model.cache_needs(), page or self.page, n_pages, slots, model.ctx.dtype, "cuda:0")
        return ModelRunner(model, cache)

    def check(self, request_tokens: dict, got: dict, what: str) -> float:
        """Every returned row against the plain implementation's row at that position. float32:
        every position within the bar. bfloat16: nine in ten of a request's positions within the
        bar, half within half of it, none beyond 0.5."""
        worst = 0.0
        bar = TOLERANCE[self.dtype]
        loose = self.dtype == "bfloat16"
        for r, rows in got.items():
            ref = self.plain_logits(request_tokens[r])
            errors = []
            for position in sorted(rows):
                err = relative_error(rows[position], ref[position])
                errors.append(err)
                assert err < (0.5 if loose else bar), (
                    f"{what}: request {r!r} differs from the plain implementation at position "
                    f"{position} of {len(request_tokens[r])}: rel error {err:.3e} (bar {bar:.0e})")
            errors.sort()
            if loose:
                assert errors[len(errors) // 2] < bar / 2, f"{what}: request {r!r}: median error {errors[len(errors) // 2]:.3e}"
                assert errors[max(0, len(errors) * 9 // 10 - 1)] < bar, f"{what}: request {r!r}: too many positions over the bar"
                worst = max(worst, errors[len(errors) // 2])
            else:
                worst = max(worst, errors[-1])
        import harness

        harness.record_error(self.dtype, "bunosun " + what, worst, bar)
        return worst
