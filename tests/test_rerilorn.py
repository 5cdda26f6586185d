"""The Rerilorn configuration, its description as parts, and the plain implementation's own
consistency (no GPU)."""

from __future__ import annotations

import pytest
import torch

import plain_rerilorn as plain
import rerilorn_tiny as rt
from pulsarlm_b200 import models  # noqa: F401  (registers the architectures)
from pulsarlm_b200.cache.manager import CacheManager
from pulsarlm_b200.config.base import ConfigError
from pulsarlm_b200.config.registry import read_model_config
from pulsarlm_b200.models.model import Model, tensor_needs_of
from pulsarlm_b200.parts.spec import KVCacheNeed, StateNeed
from pulsarlm_b200.weights.loader import check_names


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_configuration_round_trip_and_tensor_names(key):
    cfg, _ = rt.CONFIGS[key]
    arch, typed = read_model_config(cfg)
    assert arch.name == "Rerilorn" and type(typed).from_text(typed.to_text()) == typed
    assert len(typed.layers) == len(cfg["layers"])
    needs = tensor_needs_of(arch.describe(typed))
    check_names(key, needs, rt.tensor_shapes(cfg))  # (the decay's inner size is taken from the tensors)


def test_configuration_errors_name_the_key():
    cfg, _ = rt.CONFIGS["A"]
    for path, value in ((("layers", 0, "type"), "sliding"), (("layers", 1, "mlp", "kind"), "routed"),
                        (("layers", 0, "mixer", "kv_rank"), 0)):
        bad = __import__("copy").deepcopy(cfg)
        at = bad
        for step in path[:-1]:
            at = at[step]
        at[path[-1]] = value
        with pytest.raises(ConfigError) as error:
            read_model_config(bad)
        assert str(path[-1]) in str(error.value) or str(value) in str(error.value)


def test_cache_needs_of_every_holder():
    """A latent-attention layer asks for one plane of pages of its rank with its window, a
    delta-rule layer for a float32 state per head, and each input convolution for taps - 1
    rows in the engine's dtype; a layer without feed-forward has one convolution fewer."""
    cfg, _ = rt.CONFIGS["A"]
    arch, typed = read_model_config(cfg)
    model = Model(arch.describe(typed), torch.float32, torch.device("cpu"))
    needs = model.cache_needs()
    assert needs[0] == (KVCacheNeed(1, 48, 21, 5, planes=1), StateNeed((2, 72), "engine"), StateNeed((2, 72), "engine"))
    assert needs[3] == (StateNeed((3, 16, 16), "float32"), StateNeed((2, 72), "engine"))
    manager = CacheManager(needs, 16, 8, 2, torch.float32, None, allocate=False)
    assert len(manager.groups) == 1 and manager.groups[0].need.planes == 1
    assert (0, 0) in manager.layer_group and (2, 0) in manager.layer_group
    assert set(manager.state_layers) == {(0, 1), (0, 2), (1, 0), (1, 1), (1, 2), (2, 1), (3, 0), (3, 1)}
    # requests get slots and pages for every holder at once
    assert manager.open("r") == 0 and manager.reserve("r", 40) and manager.held_pages("r", 0) != []
    manager.commit("r", 40)
    assert len(manager.held_pages("r", 0)) == 2  # (window 21: the page of tokens 0..15 went back)
    manager.close("r")


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_plain_implementation_does_not_depend_on_the_cut(key):
    cfg, _ = rt.CONFIGS[key]
    weights = {n: t.double() for n, t in rt.random_weights(cfg, 2).items()}
    tokens = rt.random_tokens(cfg, 45, 3)
    whole, _ = plain.forward(cfg, weights, tokens)
    state, parts = None, []
    for lo, hi in ((0, 1), (1, 3), (3, 20), (20, 21), (21, 45)):
        out, state = plain.forward(cfg, weights, tokens[lo:hi], state)
        parts.append(out)
    assert (torch.cat(parts) - whole).abs().max() < 1e-10


def test_plain_window_and_sink():
    """One head, identity projections: a key outside the window has no weight, and the sink takes
    its share of the denominator."""
    rank = 4
    eye = torch.eye(rank, dtype=torch.float64)
    w = {"q": eye, "dkv": eye, "dkv.norm": torch.ones(rank, dtype=torch.float64), "uk": eye, "uv": eye,
         "sink": torch.tensor([0.0], dtype=torch.float64), "g": torch.zeros((1, rank), dtype=torch.float64), "o": eye}
    h = torch.tensor([[9.0, 0, 0, 0], [0, 1.0, 0, 0], [0, 0, 1.0, 0]], dtype=torch.float64)
    out, latents = plain.latent_attention_mixer(h, w, 1, rank, rank, 1.0, 2, 0.0, None)
    c = latents
    # the last token sees itself and the one before, not the first; gate = sigmoid(0) = 1/2
    s = torch.stack([c[1] @ h[2], c[2] @ h[2]])  # (queries come from h, keys from the normed latents)
    weights = torch.exp(s) / (torch.exp(s).sum() + 1.0)
    assert torch.allclose(out[2], 0.5 * (weights[0] * c[1] + weights[1] * c[2]))
    assert out[2][0] == 0.0
