"""Small Rerilorn configurations and random weights for the tests.

The configurations differ from each other in every size and constant: layer order,
widths, head counts and sizes (key size != value size, rank with and without a
tensor-core kernel), windows (one layer without), taps, eps, residual multiplier,
embedding scale, a layer without feed-forward. Weights are drawn with torch and written
with the `safetensors` package, so the engine's reader and its names are checked against
an independent file.
"""

from __future__ import annotations

import json
import os
import tempfile

import torch

import plain_rerilorn


def delta_layer(heads, dim, ff):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent_layer(heads, dim, vdim, rank, window, scale, ff):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIG_A = {
    "architecture": "Rerilorn", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "embedding": {"scale": 3.0}, "canon": {"taps": 3},
    "layers": [latent_layer(5, 8, 24, 48, 21, 0.4, 100), delta_layer(3, 16, 100),
               latent_layer(5, 8, 24, 48, 21, 0.4, None), delta_layer(3, 16, None)],
}
CONFIG_B = {
    "architecture": "Rerilorn", "vocab": 97, "width": 40, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "embedding": {"scale": 1.0}, "canon": {"taps": 5},
    "layers": [delta_layer(2, 24, 56), latent_layer(2, 12, 12, 40, None, 0.25, 56),
               latent_layer(3, 16, 8, 32, 9, 0.3, 56)],
}
CONFIG_C = {
    "architecture": "Rerilorn", "vocab": 128, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
    "embedding": {"scale": 8.0}, "canon": {"taps": 2},
    "layers": [latent_layer(4, 16, 16, 64, 40, 0.25, 96), delta_layer(1, 64, 96), latent_layer(8, 8, 16, 96, 17, 0.35, 96)],
}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 32), "C": (CONFIG_C, 16)}
DECAY_RANK = 6


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (w,)
        if cfg.get("canon"):
            shapes[p + "canon1"] = (w, cfg["canon"]["taps"])
        if layer["type"] == "general_delta":
            hd = m["heads"] * m["dim"]
            for name in ("r", "k", "v", "g", "a"):
                shapes[p + "mix." + name] = (hd, w)
            for name in ("a.b", "w0", "norm"):
                shapes[p + "mix." + name] = (hd,)
            shapes[p + "mix.w1"] = (DECAY_RANK, w)
            shapes[p + "mix.w2"] = (hd, DECAY_RANK)
            shapes[p + "mix.o"] = (w, hd)
        else:
            h, d, vd, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            shapes[p + "mix.q"] = (h * d, w)
            shapes[p + "mix.dkv"] = (r, w)
            shapes[p + "mix.dkv.norm"] = (r,)
            shapes[p + "mix.uk"] = (h * d, r)
            shapes[p + "mix.uv"] = (h * vd, r)
            shapes[p + "mix.sink"] = (h,)
            shapes[p + "mix.g"] = (h, w)
            shapes[p + "mix.o"] = (w, h * vd)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (w,)
            if cfg.get("canon"):
                shapes[p + "canon2"] = (w, cfg["canon"]["taps"])
            shapes[p + "mlp.up"], shapes[p + "mlp.up.b"] = (ff, w), (ff,)
            shapes[p + "mlp.down"], shapes[p + "mlp.down.b"] = (w, ff), (w,)
    return shapes


def random_weights(cfg: dict, seed: int, dtype: torch.dtype = torch.float32) -> dict:
    """Matrices N(0, 1/sqrt(in)) (queries and keys twice that, so that attention is far from
    uniform), norm scales 1 + 0.1 N, biases and sinks N(0, 0.5), convolution taps N(0, 0.4);
    rounded to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if leaf in ("norm1", "norm1b", "norm2", "norm2b", "mix.norm", "mix.dkv.norm", "final.norm") or name == "final.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        elif leaf in ("canon1", "canon2"):
            t = 0.4 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen) / cfg["embedding"]["scale"]
        else:
            gain = 2.0 if leaf in ("mix.q", "mix.uk", "mix.k", "mix.r") else 1.0
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
# float64. The float32 engine is the sharp comparison (worst seen 2e-6). In bfloat16 the engine rounds
# a sublayer's activations at some ten places and the out-norms rescale what was rounded; the worst seen
# over these models is 5.4e-2, so the bfloat16 runs catch what breaks a schedule, and what is off by a
# rounding is left to the float32 runs, to the kernels' own tests with a key made to dominate, and to
# the comparison of the tensor-core path with the CUDA-core path (1e-2).
TOLERANCE = {"float32": 2e-4, "bfloat16": 8e-2}


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max())


class TinyRerilorn:
    """A configuration with random weights rounded to the engine's dtype (so that the plain
    implementation, which runs in float64, and the engine start from identical numbers),
    its model folder, and the plain implementation's logits on demand."""

    def __init__(self, key: str, dtype: str, seed: int = 1, cfg: dict | None = None, weights: dict | None = None):
        self.cfg, self.page = CONFIGS[key] if cfg is None else (cfg, 16)
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
            self._plain[key] = plain_rerilorn.forward(self.cfg, self.plain_weights, list(tokens))[0]
        return self._plain[key]

    def rounding_error(self, tokens) -> torch.Tensor:
        """Per position, the error (as `relative_error` measures it) of the plain implementation
        when nothing but its norms' outputs are rounded to bfloat16: how touchy each position of
        this model is to roundings. Some positions of small random models are: a bfloat16 engine,
        which rounds at more places, cannot be held to a flat bar there."""
        key = ("rounded",) + tuple(tokens)
        if key not in self._plain:
            exact = self.plain_logits(tokens)
            plain_norm = plain_rerilorn.rms_norm
            plain_rerilorn.rms_norm = lambda x, weight, eps: plain_norm(x, weight, eps).to(torch.bfloat16).double()
            try:
                rounded = plain_rerilorn.forward(self.cfg, self.plain_weights, list(tokens))[0]
            finally:
                plain_rerilorn.rms_norm = plain_norm
            self._plain[key] = torch.tensor([relative_error(rounded[i], exact[i]) for i in range(len(tokens))])
        return self._plain[key]

    def runner(self, n_pages: int, slots: int = 4, page: int | None = None):
        from pulsarlm_b200.cache.manager import CacheManager
        from pulsarlm_b200.engine.loading import load_model
        from pulsarlm_b200.engine.runner import ModelRunner

        model = load_model(self.folder, self.dtype, "cuda:0")
        cache = CacheManager(model.cache_needs(), page or self.page, n_pages, slots, model.ctx.dtype, "cuda:0")
        return ModelRunner(model, cache)

    def check(self, request_tokens: dict, got: dict, what: str, touchy: bool = False) -> float:
        """Every returned row against the plain implementation's row at that position. touchy (for
        models drawn at random, in bfloat16, some of which amplify a rounding several times at a
        few positions, as `rounding_error` shows without any engine): half of a request's
        positions within half the bar, nine in ten within the bar, none beyond 0.5; the same
        models are held to the float32 bar at every position first."""
        worst = 0.0
        bar = TOLERANCE[self.dtype]
        loose = touchy and self.dtype == "bfloat16"
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
                assert errors[len(errors) * 9 // 10 - 1] < bar, f"{what}: request {r!r}: too many positions over the bar"
                worst = max(worst, errors[len(errors) // 2])
            else:
                worst = max(worst, errors[-1])
        import harness

        harness.record_error(self.dtype, "rerilorn " + what, worst, bar)
        return worst
