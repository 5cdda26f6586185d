"""The Bunosun decoder's configuration, description and plain implementation, on the CPU."""

from __future__ import annotations

import json

import pytest
import torch

import bunosun_tiny as bt
import plain_bunosun as plain
from pulsarlm_b200.config.base import ConfigError
from pulsarlm_b200.config.registry import read_model_config, registered_architectures
from pulsarlm_b200.models.model import tensor_needs_of


def test_the_architecture_is_registered():
    assert "Bunosun" in registered_architectures()


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_configuration_round_trip_and_tensor_names(key):
    cfg_text, _ = bt.CONFIGS[key]
    arch, cfg = read_model_config(cfg_text)
    assert arch.name == "Bunosun"
    assert arch.read_config(cfg.to_text()) == cfg
    assert arch.read_config(json.loads(json.dumps(cfg.to_text()))) == cfg
    needs = tensor_needs_of(arch.describe(cfg))
    shapes = bt.tensor_shapes(cfg_text)
    assert set(needs) == set(shapes)
    for name, need in needs.items():
        assert all(a in (-1, b) for a, b in zip(need.shape, shapes[name])), name


def test_the_order_of_runs():
    _, cfg = read_model_config(bt.CONFIG_A)
    assert cfg.runs() == ([0, 1, 2, 1, 2, 3], [3])
    _, cfg = read_model_config(bt.CONFIG_B)
    assert cfg.runs() == ([0, 1, 2], [])
    _, cfg = read_model_config(bt.CONFIG_C)
    assert cfg.runs() == ([0, 1, 0, 1, 0, 1], [2, 4])
    for text in (bt.CONFIG_A, bt.CONFIG_B, bt.CONFIG_C):
        order, again = read_model_config(text)[1].runs()
        want_order, want_again = plain.run_order(text)
        assert order == want_order and set(again) == want_again
    arch, cfg = read_model_config(bt.CONFIG_C)
    spec = arch.describe(cfg)
    assert spec.cache_per_run and spec.order == [0, 1, 0, 1, 0, 1] and spec.rejoin_runs == (2, 4)


def test_bad_configurations_are_refused():
    def broken(change):
        text = json.loads(json.dumps(bt.CONFIG_A))
        change(text)
        with pytest.raises(ConfigError):
            read_model_config(text)

    broken(lambda t: t["layers"][0].update(type="other"))
    broken(lambda t: t["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda t: t["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda t: t["layers"][0]["mlp"]["router"].update(top=5))        # more than the kept groups hold
    broken(lambda t: t["layers"][0]["mlp"]["router"]["groups"].update(count=3))
    broken(lambda t: t["loop"].update(stop=9))
    broken(lambda t: t["layers"][1]["mixer"].pop("conv"))
    broken(lambda t: t.pop("norm"))


def test_plain_rotation_turns_neighbours_and_keeps_the_rest():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    y = plain.rotate_pairs(x, torch.arange(5), 4, 100.0, 2.0)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.equal(y[0], x[0])
    assert torch.allclose((y[..., 0:4:2] ** 2 + y[..., 1:4:2] ** 2), (x[..., 0:4:2] ** 2 + x[..., 1:4:2] ** 2))
    angle = 3 * 100.0 ** (-2.0 / 4) / 2.0   # position 3, pair 1
    assert torch.allclose(y[3, :, 2], x[3, :, 2] * torch.cos(torch.tensor(angle)) - x[3, :, 3] * torch.sin(torch.tensor(angle)))


def test_plain_window_and_router():
    see = plain.visible(6, 3)
    assert see[5].tolist() == [False, False, False, True, True, True] and see[1].tolist() == [True, True] + [False] * 4
    # a group shut out stays out even when its experts' scores are the largest after the kept group's best
    w = {"r.router": torch.eye(4, dtype=torch.float64) * 8, "r.correction": torch.tensor([0.0, -5.0, 0.0, 0.0], dtype=torch.float64)}
    mlp = {"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}}
    h = torch.tensor([[1.0, 0.0, 0.5, 0.4]], dtype=torch.float64)
    chosen, weights = plain.route(mlp, w, "r.", h)
    assert chosen.tolist() == [[0, 1]] and abs(float(weights.sum()) - 1.0) < 1e-12


def test_plain_prefix_does_not_depend_on_what_follows():
    cfg, _ = bt.CONFIGS["A"]
    weights = {k: v.double() for k, v in bt.random_weights(cfg, 2).items()}
    tokens = bt.random_tokens(cfg, 40, 3)
    whole = plain.forward(cfg, weights, tokens)[0]
    part = plain.forward(cfg, weights, tokens[:17])[0]
    assert torch.allclose(whole[:17], part, atol=1e-9)
