"""The Bunosun decoder in the engine against the plain implementation (plain_bunosun.py):
each mechanism's kernel alone, then whole models under every kind of schedule."""

from __future__ import annotations

import json

import pytest
import torch

import bunosun_tiny as bt
import harness
import plain_bunosun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from pulsarlm_b200.kernels import ops

    ops.require_device()
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# --------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 72, 1032])
def test_pair_residual_and_both_norms(dtype, width):
    ops = _ops()
    gen = torch.Generator().manual_seed(width)
    rows = 9
    x = torch.randn(rows, width, generator=gen)
    y1, y2 = (torch.randn(rows, width, generator=gen).to(dtype) for _ in range(2))
    s1, s2, w1, w2 = (torch.randn(width, generator=gen) for _ in range(4))
    also = torch.randn(rows, width, generator=gen)
    for use_y2, use_also in ((True, True), (False, False), (True, False)):
        want_x = x.double() + y1.double() * s1.double()
        if use_y2:
            want_x = want_x + y2.double() * s2.double()
        if use_also:
            want_x = want_x + also.double()
        xd = x.to(DEV).clone()
        h1 = torch.empty(rows, width, dtype=dtype, device=DEV)
        h2 = torch.empty(rows, width, dtype=dtype, device=DEV)
        ops.pair_residual_norm(xd, y1.to(DEV), s1.to(DEV), y2.to(DEV) if use_y2 else None, s2.to(DEV) if use_y2 else None,
                               also.to(DEV) if use_also else None, w1.to(DEV), w2.to(DEV), h1, h2, 1e-5)
        bar = 1e-5 if dtype == torch.float32 else 1e-2
        assert bt.relative_error(xd.cpu(), want_x) < 1e-6
        assert bt.relative_error(h1.cpu(), plain.rms(want_x, 1e-5) * w1.double()) < bar
        assert bt.relative_error(h2.cpu(), plain.rms(want_x, 1e-5) * w2.double()) < bar
        # the row-gather form leaves the stream as it is
        xd2 = x.to(DEV).clone()
        picked = torch.empty(2, width, dtype=dtype, device=DEV)
        ops.pair_residual_norm(xd2, y1.to(DEV), s1.to(DEV), None, None, None, w1.to(DEV), None, picked, None, 1e-5,
                               _i32([7, 2]))
        assert torch.equal(xd2.cpu(), x)
        want = plain.rms(x.double() + y1.double() * s1.double(), 1e-5) * w1.double()
        assert bt.relative_error(picked.cpu(), want[[7, 2]]) < bar


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_with_activation_over_columns_of_a_wider_matrix(taps, dtype):
    """Two sequences in portions of unequal sizes (also shorter than the taps); the rows are columns
    of a wider matrix, as a mixer's stacked projection leaves them."""
    ops = _ops()
    gen = torch.Generator().manual_seed(taps)
    width, extra = 40, 12
    lengths = {0: 23, 1: 9}
    full = {e: torch.randn(n, width + extra, generator=gen).to(dtype) for e, n in lengths.items()}
    weight = (0.5 * torch.randn(width, taps, generator=gen))
    want = {e: plain.causal_conv_silu(full[e][:, :width].double(), weight.double()) for e in lengths}
    state = torch.zeros(3, max(taps - 1, 0), width, dtype=dtype, device=DEV)
    fed = {0: 0, 1: 0}
    got = {e: [] for e in lengths}
    for parts in ([(0, 1), (1, 2)], [(1, 1), (0, 5)], [(0, 2)], [(0, 15), (1, 6)]):
        rows = torch.cat([full[e][fed[e]: fed[e] + n] for e, n in parts]).to(DEV)
        entry = _i32([i for i, (_, n) in enumerate(parts) for _ in range(n)])
        slots = _i32([2 - e for e, _ in parts])
        out = torch.empty(rows.shape[0], width, dtype=dtype, device=DEV)
        ops.short_conv_act(rows[:, :width], weight.to(DEV), state, entry, slots, out, residual=False, act="silu")
        if taps > 1:
            ops.short_conv_state_strided(rows[:, :width], entry, slots, state)
        at = 0
        for e, n in parts:
            got[e].append(out[at: at + n].cpu())
            at += n
            fed[e] += n
    for e in lengths:
        assert fed[e] == lengths[e]
        assert bt.relative_error(torch.cat(got[e]), want[e]) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("taps", [2, 4, 6])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_and_state_in_one_launch_for_single_tokens(taps, dtype):
    """Three sequences fed a token a step: the result equals the two-kernel path's bit for bit."""
    ops = _ops()
    gen = torch.Generator().manual_seed(taps)
    width, extra, steps = 48, 8, 9
    full = torch.randn(steps, 3, width + extra, generator=gen).to(dtype).to(DEV)
    weight = (0.5 * torch.randn(width, taps, generator=gen)).to(DEV)
    states = [torch.zeros(4, taps - 1, width, dtype=dtype, device=DEV) for _ in range(2)]
    entry, slots = _i32([0, 1, 2]), _i32([3, 0, 2])
    for step in range(steps):
        rows = full[step]
        outs = [torch.empty(3, width, dtype=dtype, device=DEV) for _ in range(2)]
        assert ops.short_conv_single(rows[:, :width], weight, states[0], entry, slots, outs[0], residual=False, act="silu")
        ops.short_conv_act(rows[:, :width], weight, states[1], entry, slots, outs[1], residual=False, act="silu")
        ops.short_conv_state_strided(rows[:, :width], entry, slots, states[1])
        assert torch.equal(outs[0], outs[1]) and torch.equal(states[0], states[1])
    want = plain.causal_conv_silu(full[:, 1, :width].double().cpu(), weight.double().cpu())
    assert bt.relative_error(outs[0][1].cpu(), want[-1]) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("heads,qk_heads,dim,vdim", [(1, 1, 8, 8), (4, 2, 16, 24), (2, 1, 64, 32), (3, 3, 24, 40),
                                                     (2, 2, 128, 128), (1, 1, 40, 200)])
def test_gated_delta_kernel(heads, qk_heads, dim, vdim):
    """The recurrence and its finish against the plain scan, two sequences in unequal portions with
    the state carried between steps in slots that are not the entries' numbers."""
    ops = _ops()
    gen = torch.Generator().manual_seed(dim + vdim)
    lengths = {0: 37, 1: 12}
    data, want = {}, {}
    a_log = 0.5 * torch.randn(heads, generator=gen)
    dt_bias = 0.5 * torch.randn(heads * dim, generator=gen)
    norm = 1.0 + 0.1 * torch.randn(vdim, generator=gen)
    for e, n in lengths.items():
        q, k = (torch.randn(n, qk_heads * dim, generator=gen) for _ in range(2))
        v = torch.randn(n, heads * vdim, generator=gen)
        b_pre = torch.randn(n, heads, generator=gen)
        a_pre = torch.randn(n, heads * dim, generator=gen)
        gate_pre = torch.randn(n, heads * vdim, generator=gen)
        data[e] = (q, k, v, b_pre, a_pre, gate_pre)
        qd, kd = q.double().view(n, qk_heads, dim), k.double().view(n, qk_heads, dim)
        qd = qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        kd = kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(
            a_pre.double() + dt_bias.double()).view(n, heads, dim))
        o = plain.delta_scan(qd, kd, v.double().view(n, heads, vdim), torch.sigmoid(b_pre.double()), decay)
        want[e] = (plain.rms(o, 1e-5) * norm.double() * torch.sigmoid(gate_pre.double()).view(n, heads, vdim)).reshape(n, -1)
    state = torch.zeros(4, heads, dim, vdim, dtype=torch.float32, device=DEV)
    fed = {0: 0, 1: 0}
    got = {e: [] for e in lengths}
    for parts in ([(0, 20), (1, 1)], [(1, 2), (0, 1)], [(0, 16), (1, 9)]):
        stacked = [torch.cat([data[e][i][fed[e]: fed[e] + n] for e, n in parts]).to(DEV) for i in range(6)]
        qkv = torch.cat(stacked[:3], dim=1)  # (q, k and v are columns of one matrix, as the convolution leaves them)
        stacked[:3] = [qkv[:, :qk_heads * dim], qkv[:, qk_heads * dim:2 * qk_heads * dim], qkv[:, 2 * qk_heads * dim:]]
        first, at = [], 0
        for _, n in parts:
            first.append(at)
            at += n
        out = torch.empty(at, heads * vdim, dtype=torch.float32, device=DEV)
        ops.gated_delta(*stacked, a_log.to(DEV), dt_bias.to(DEV), norm.to(DEV), state, _i32(first),
                        _i32([n for _, n in parts]), _i32([3 - e for e, _ in parts]), out, heads, qk_heads, dim, vdim,
                        1e-6, dim ** -0.5, 1e-5)
        for (e, n), f in zip(parts, first):
            got[e].append(out[f: f + n].cpu())
            fed[e] += n
    for e in lengths:
        assert bt.relative_error(torch.cat(got[e]), want[e]) < 2e-5


@pytest.mark.parametrize("experts,top,groups,keep", [(8, 2, 4, 2), (6, 1, 1, 1), (12, 3, 3, 2), (64, 6, 8, 3), (5, 5, 1, 1)])
def test_router_chooses_as_the_plain_one(experts, top, groups, keep):
    """Scores, correction (large: choice scores go negative), groups shut out, ties aside."""
    ops = _ops()
    gen = torch.Generator().manual_seed(experts)
    hidden, tokens = 48, 200
    h = torch.randn(tokens, hidden, generator=gen)
    w = {"r.router": torch.randn(experts, hidden, generator=gen) * 0.3, "r.correction": torch.randn(experts, generator=gen) - 1.0}
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    chosen, weights = plain.route(mlp, {k: v.double() for k, v in w.items()}, "r.", h.double())
    ids, got = ops.moe_route(h.to(DEV), w["r.router"].to(DEV), w["r.correction"].to(DEV), top, groups, keep)
    assert torch.equal(ids.cpu().long(), chosen)
    assert bt.relative_error(got.cpu(), weights) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top", [(1, 10, 3), (7, 10, 3), (150, 10, 3), (50, 80, 1), (300, 5, 5)])
def test_routed_experts_pair_by_pair_and_grouped(dtype, tokens, experts, top, monkeypatch):
    """The part alone: few tokens stream their experts' weights; many (bfloat16) are sorted by expert
    (also with more experts than tokens, so that most experts get no row, and with every expert chosen)."""
    from pulsarlm_b200.parts import moe as moe_part
    from pulsarlm_b200.parts.registry import BuildContext
    from pulsarlm_b200.parts.spec import PartSpec

    _ops()
    gen = torch.Generator().manual_seed(tokens)
    hidden, ff = 64, 40
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": 5, "keep": 3 if top < 5 else 5}}, "shared": {"ff": 24}}
    w = {"m.router": torch.randn(experts, hidden, generator=gen) * 0.5, "m.correction": 0.1 * torch.randn(experts, generator=gen)}
    for name, size in [(f"e{e}", ff) for e in range(experts)] + [("shared", 24)]:
        w[f"m.{name}.gate"] = (torch.randn(size, hidden, generator=gen) / hidden ** 0.5).to(dtype)
        w[f"m.{name}.up"] = (torch.randn(size, hidden, generator=gen) / hidden ** 0.5).to(dtype)
        w[f"m.{name}.down"] = (torch.randn(hidden, size, generator=gen) / size ** 0.5).to(dtype)
    h = torch.randn(tokens, hidden, generator=gen).to(dtype)
    want = plain.routed_experts(mlp, {k: v.double() for k, v in w.items()}, "m.", h.double())
    spec = PartSpec("moe", {"hidden_size": hidden, "expert_size": ff, "n_experts": experts, "top": top, "groups": 5,
                            "keep_groups": mlp["router"]["groups"]["keep"], "shared_size": 24},
                    {"router": "m.router", "correction": "m.correction", "expert_gate": "m.e{e}.gate",
                     "expert_up": "m.e{e}.up", "expert_down": "m.e{e}.down", "shared_gate": "m.shared.gate",
                     "shared_up": "m.shared.up", "shared_down": "m.shared.down"})
    part = moe_part.RoutedExperts(spec, BuildContext(dtype, torch.device(DEV)))
    part.load({k: v.to(DEV) for k, v in w.items()})
    got = part.forward(h.to(DEV), None)
    assert bt.relative_error(got.cpu(), want) < (1e-5 if dtype == torch.float32 else 2e-2)
    if dtype == torch.bfloat16 and tokens >= moe_part.GROUPED_MIN_TOKENS:
        monkeypatch.setattr(moe_part, "GROUPED_MIN_TOKENS", 10 ** 9)
        assert bt.relative_error(part.forward(h.to(DEV), None).cpu(), want) < 2e-2


# --------------------------------------------------------------------------- whole models
def _model(key, dtype, seed=1):
    return bt.TinyBunosun(key, dtype, seed)


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_their_first_tokens(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": bt.random_tokens(tm.cfg, 75, 3), "q": bt.random_tokens(tm.cfg, 5, 4), "r": bt.random_tokens(tm.cfg, 1, 5)}
    got = harness.replay(runner, [([("p", tokens["p"], list(range(75)))], ["p"]),
                                  ([("q", tokens["q"], list(range(5)))], ["q"]), ([("r", tokens["r"], [0])], ["r"])])
    tm.check(tokens, got, f"{key} whole")


def test_the_stream_after_every_layer_run():
    """float32, the residual stream after each run of each layer (a repeated layer counts every
    time) against the plain implementation's."""
    from pulsarlm_b200.engine.runner import StepEntry

    tm = _model("A", "float32")
    runner = tm.runner(8)
    tokens = bt.random_tokens(tm.cfg, 20, 9)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def spy(x, delta, batch, inner=inner):
            x, pending = inner(x, delta, batch)
            full = x.double() + pending.y1.double() * pending.s1.double()
            if pending.y2 is not None:
                full = full + pending.y2.double() * pending.s2.double()
            seen.append(full.cpu())
            return x, pending

        block.forward = spy
    runner.step([StepEntry("p", tokens, [19])])
    _, streams = plain.forward(tm.cfg, tm.plain_weights, tokens)
    assert len(seen) == len(streams) == 6
    for got, want in zip(seen, streams):
        assert bt.relative_error(got, want) < 1e-5


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(key, dtype):
    """A prompt in one step, then 70 tokens one by one: past every window and over page borders."""
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": bt.random_tokens(tm.cfg, 110, 5)}
    steps = [([("p", tokens["p"][:40], [0, 1, 39])], [])]
    steps += [([("p", [tokens["p"][i]], [0])], []) for i in range(40, 110)]
    tm.check(tokens, harness.replay(runner, steps), f"{key} decode")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_by_token_from_the_start(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(8)
    tokens = {"p": bt.random_tokens(tm.cfg, 30, 6)}
    steps = [([("p", [t], [0])], []) for t in tokens["p"]]
    tm.check(tokens, harness.replay(runner, steps), f"{key} from the start")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": bt.random_tokens(tm.cfg, 150, 7)}
    cuts = [2, 2, 3, 1, 1, 7, 16, 2, 33, 1, 2, 17, 31, 2, 30]
    assert sum(cuts) == 150
    steps, at = [], 0
    for n in cuts:
        steps.append(([("p", tokens["p"][at: at + n], list(range(n)))], []))
        at += n
    tm.check(tokens, harness.replay(runner, steps), f"{key} portions")


def test_float32_bits_do_not_depend_on_the_cut():
    """In float32 every kernel adds in an order fixed by the token's own place: logits of a prompt
    fed whole and fed in portions are equal bit for bit."""
    tm = _model("A", "float32")
    tokens = bt.random_tokens(tm.cfg, 90, 8)
    whole = harness.replay(tm.runner(12), [([("p", tokens, list(range(90)))], [])])["p"]
    steps, at = [], 0
    for n in [5, 1, 2, 40, 1, 1, 3, 37]:
        steps.append(([("p", tokens[at: at + n], list(range(n)))], []))
        at += n
    cut = harness.replay(tm.runner(12), steps)["p"]
    for position in range(90):
        assert torch.equal(whole[position], cut[position]), position


@pytest.mark.parametrize("key", ["A", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_and_reused_pages_and_slots(key, dtype):
    """Up to three live requests of unequal lengths, portions beside single tokens, requests
    that pause, end and are followed by new ones in the same slots and pages (the pool is as small
    as the schedule allows)."""
    tm = _model(key, dtype)
    page = tm.page
    runner = tm.runner(3 * (-(-100 // page) + 1), slots=3)
    lengths = {"a": 100, "b": 37, "c": 64, "d": 90, "e": 3, "f": 45}
    tokens = {r: bt.random_tokens(tm.cfg, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    fed = {r: 0 for r in lengths}

    def take(r, n):
        n = min(n, lengths[r] - fed[r])
        part = tokens[r][fed[r]: fed[r] + n]
        fed[r] += n
        return (r, part, list(range(n)))

    steps = []

    def step(*parts):
        entries = [take(r, n) for r, n in parts if fed[r] < lengths[r]]
        ends = [r for r, _, _ in entries if fed[r] == lengths[r]]
        if entries:
            steps.append((entries, ends))

    step(("a", 30), ("b", 2))
    step(("a", 1), ("b", 33), ("c", 17))
    step(("b", 1), ("c", 2))
    step(("a", 50), ("b", 1))            # b ends: its slot and pages go to d
    step(("a", 1), ("c", 40), ("d", 16))
    for _ in range(6):
        step(("a", 1), ("c", 1), ("d", 1))
    step(("a", 19), ("d", 2))            # a ends
    step(("c", 5), ("d", 60), ("e", 3))  # c, e end (e within one step)
    step(("d", 11), ("f", 44))
    step(("d", 1), ("f", 1))
    assert all(fed[r] == lengths[r] for r in lengths)
    got = harness.replay(runner, steps)
    tm.check(tokens, got, f"{key} mixed")
    stats = runner.cache.stats()
    assert stats["slots_used"] == 0 and all(g["used"] == 0 for g in stats["groups"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_equals_each_request_alone(dtype):
    tm = _model("C", dtype)
    tokens = {r: bt.random_tokens(tm.cfg, n, 20 + i) for i, (r, n) in enumerate({"a": 50, "b": 9, "c": 33}.items())}
    alone = {}
    for r, t in tokens.items():
        alone.update(harness.replay(tm.runner(8), [([(r, t[:-3], [len(t) - 4])], [])] +
                                    [([(r, [t[i]], [0])], []) for i in range(len(t) - 3, len(t))]))
    runner = tm.runner(16)
    steps = [([(r, t[:-3], [len(t) - 4]) for r, t in tokens.items()], [])]
    steps += [([(r, [t[len(t) - 3 + i]], [0]) for r, t in tokens.items()], []) for i in range(3)]
    together = harness.replay(runner, steps)
    for r in tokens:
        for position, row in alone[r].items():
            if dtype == "float32":
                assert torch.equal(row, together[r][position])
            else:
                assert bt.relative_error(together[r][position], row) < 6e-2


def _peaked(window, dtype, rot_dims=8):
    """One attention layer whose queries and keys are scaled up until nearly all of a map's weight
    sits on one key: a key wrongly seen or missed at the window's edge then moves the logits by
    far more than any bar."""
    cfg = {"architecture": "Bunosun", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [bt.attention_layer(2, 1, 16, 32, window, rot_dims, None, diff=0.4, scale=0.25, factor=1.5)]}
    weights = bt.random_weights(cfg, 7, torch.float32 if dtype == "float32" else torch.bfloat16)
    for name in ("l0.mix.q", "l0.mix.k"):
        weights[name] = weights[name] * 3.0
    return bt.TinyBunosun("-", dtype, cfg=cfg, weights=weights)


@pytest.mark.parametrize("window", [1, 16, 23, 50])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_windows_edge_in_prompts_and_decoding(window, dtype):
    tm = _peaked(window, dtype)
    tokens = {"p": bt.random_tokens(tm.cfg, 140, 11), "d": bt.random_tokens(tm.cfg, 140, 12)}
    # the plain implementation itself must tell a window of one more or one less apart
    for other in (window + 1, max(1, window - 1)):
        if other != window:
            cfg = json.loads(json.dumps(tm.cfg))
            cfg["layers"][0]["mixer"]["mask"]["size"] = other
            moved = plain.forward(cfg, tm.plain_weights, tokens["p"])[0]
            assert bt.relative_error(moved, tm.plain_logits(tokens["p"])) > 0.05
    steps = [([("p", tokens["p"], list(range(140)))], ["p"]), ([("d", tokens["d"][:5], [4])], [])]
    steps += [([("d", [tokens["d"][i]], [0])], []) for i in range(5, 140)]
    got = harness.replay(tm.runner(24), steps)
    for r in tokens:
        ref = tm.plain_logits(tokens[r])
        for position, row in got[r].items():
            assert bt.relative_error(row, ref[position]) < (2e-4 if dtype == "float32" else 0.1), (r, position)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    tm = _model("B", dtype)
    runner = tm.runner(16)
    tokens = {"p": bt.random_tokens(tm.cfg, 400, 30)}
    steps = [([("p", tokens["p"][:4], [3])], [])]
    steps += [([("p", [tokens["p"][i]], [0] if i % 9 == 0 or i > 390 else [])], []) for i in range(4, 400)]
    tm.check(tokens, harness.replay(runner, steps), "B long decoding")


def test_a_far_token_reaches_through_the_recurrence():
    """Two prompts that differ in their first token only, in a model whose attention sees four
    tokens and whose recurrent layer forgets slowly (a small decay rate): 90 tokens on, far past the
    windows' reach, the logits still differ, and the engine reproduces that difference."""
    cfg = {"architecture": "Bunosun", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [bt.attention_layer(2, 2, 8, 16, 4, 4, None), bt.delta_layer(2, 1, 16, 24, 3, bt.moe(4, 2, 24))]}
    weights = bt.random_weights(cfg, 5)
    weights["l1.mix.A_log"] = torch.full_like(weights["l1.mix.A_log"], -7.0)
    tm = bt.TinyBunosun("-", "float32", cfg=cfg, weights=weights)
    base = bt.random_tokens(cfg, 91, 40)
    other = [(base[0] + 1) % cfg["vocab"]] + base[1:]
    tokens = {"x": base, "y": other}
    got = harness.replay(tm.runner(16), [([("x", base, [90]), ("y", other, [90])], ["x", "y"])])
    tm.check(tokens, got, "far token")
    want = tm.plain_logits(base)[90] - tm.plain_logits(other)[90]
    assert want.abs().max() > 1e-3 * tm.plain_logits(base)[90].abs().max()
    assert bt.relative_error(got["x"][90] - got["y"][90], want) < 0.05


def test_sizes_come_from_the_configuration():
    """Constants that a given model may leave at 1 or equal to one another: one head, one expert
    of which one is chosen, one group, one tap (no convolution state), a window of one, a loop that
    runs once, an embedding scale of 1, map, value and state sizes all equal."""
    cfg = {
        "architecture": "Bunosun", "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
        "layers": [bt.attention_layer(1, 1, 16, 16, 1, 16, bt.moe(1, 1, 24), diff=0.2, scale=0.5),
                   bt.delta_layer(1, 1, 16, 16, 1, bt.moe(4, 4, 16, 2, 2)),
                   bt.attention_layer(2, 2, 8, 24, 2, 4, None, diff=0.7, scale=1.0, base=50.0)],
        "loop": {"start": 1, "stop": 2, "times": 1},
    }
    for dtype in ("float32", "bfloat16"):
        tm = bt.TinyBunosun("-", dtype, cfg=cfg)
        tokens = {"p": bt.random_tokens(cfg, 40, 50)}
        steps = [([("p", tokens["p"][:20], list(range(20)))], [])]
        steps += [([("p", [t], [0])], []) for t in tokens["p"][20:]]
        tm.check(tokens, harness.replay(tm.runner(8), steps), "sizes of one")


def _random_config(seed: int) -> dict:
    """Sizes, constants, layer order and loop drawn at random: widths that are no multiple of 8,
    odd head counts and groups, map and value sizes with and without a tensor-core kernel, windows
    from 1 up, layers with and without feed-forward, window or rotation."""
    gen = torch.Generator().manual_seed(seed)

    def pick(options):
        return options[int(torch.randint(0, len(options), (1,), generator=gen))]

    width = pick([36, 52, 64, 100, 136])
    layers = []
    n_layers = pick([2, 3, 4])
    for _ in range(n_layers):
        experts, groups = pick([(4, 2), (6, 3), (8, 1), (9, 3), (16, 4)])
        keep = pick(list(range(1, groups + 1)))
        top = pick(list(range(1, min(4, keep * (experts // groups)) + 1)))
        mlp = pick([None, bt.moe(experts, top, pick([24, 40, 72]), groups, keep, pick([None, 16, 56]))])
        kv = pick([1, 2, 3])
        heads = kv * pick([1, 2, 3])
        if pick([0, 1, 1]) == 0:
            layers.append(bt.delta_layer(heads, kv, pick([8, 16, 24, 40, 64]), pick([8, 16, 24, 48]), pick([1, 2, 3, 4, 5]), mlp))
        else:
            dim = pick([8, 12, 16, 24, 32, 40, 64])
            layers.append(bt.attention_layer(heads, kv, dim, pick([8, 16, 24, 40, 64, 2 * dim]),
                                             pick([None, 1, 2, 5, 16, 17, 31, 33, 50]), pick([0, 2, 4, dim]), mlp,
                                             diff=pick([0.1, 0.5, 0.8]), scale=pick([0.2, 0.35, dim ** -0.5]),
                                             base=pick([100.0, 10000.0]), factor=pick([1.0, 2.0, 8.0])))
    start = pick(list(range(n_layers)))
    stop = pick(list(range(start, n_layers + 1)))
    return {"architecture": "Bunosun", "vocab": pick([64, 101, 257]), "width": width,
            "norm": {"eps": pick([1e-6, 1e-5, 1e-3])}, "embedding": {"scale": pick([1.0, 2.5, width ** 0.5])},
            "layers": layers, "loop": {"start": start, "stop": stop, "times": pick([1, 2, 3])}}


@pytest.mark.parametrize("seed", list(range(10)))
def test_configurations_drawn_at_random(seed):
    """Each drawn model under a mixed schedule (portions, single tokens, a request that ends and one
    that takes its slot), float32 against the plain implementation at the float32 bar, then bfloat16
    at its own."""
    cfg = _random_config(seed)
    page = [16, 32, 64][seed % 3]
    for dtype in ("float32", "bfloat16"):
        tm = bt.TinyBunosun("-", dtype, seed=seed, cfg=cfg)
        tokens = {r: bt.random_tokens(cfg, n, 100 + seed + i) for i, (r, n) in enumerate({"a": 70, "b": 23, "c": 41}.items())}
        a, b, c = tokens["a"], tokens["b"], tokens["c"]
        steps = [([("a", a[:35], list(range(35))), ("b", b[:2], [0, 1])], []),
                 ([("a", a[35:36], [0]), ("b", b[2:23], list(range(21)))], ["b"]),
                 ([("a", a[36:37], [0]), ("c", c[:3], [0, 1, 2])], []),
                 ([("c", c[3:40], list(range(37))), ("a", a[37:38], [0])], [])]
        steps += [([("a", [a[i]], [0])] + ([("c", [c[40]], [0])] if i == 38 else []), ["c"] if i == 38 else [])
                  for i in range(38, 70)]
        runner = tm.runner(-(-70 // page) + -(-41 // page) + 2, slots=2, page=page)
        tm.check(tokens, harness.replay(runner, steps), f"random configuration {seed}")


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(8, 1, 16, 32), (10, 1, 8, 16), (4, 4, 64, 128), (2, 1, 72, 96),
                                                     (1, 1, 128, 256)])
def test_head_counts_and_row_sizes_with_and_without_a_tensor_core_kernel(heads, kv_heads, dim, vdim):
    """Sixteen and twenty query rows per kv head, rows of 128, of 144 and of 256: prompts, portions and
    single tokens in bfloat16 and float32."""
    cfg = {"architecture": "Bunosun", "vocab": 71, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [bt.attention_layer(heads, kv_heads, dim, vdim, 37, min(dim, 8), None, diff=0.4,
                                         scale=dim ** -0.5, factor=2.0)]}
    for dtype in ("float32", "bfloat16"):
        tm = bt.TinyBunosun("-", dtype, cfg=cfg, seed=3)
        tokens = {"p": bt.random_tokens(cfg, 100, 60), "q": bt.random_tokens(cfg, 20, 61)}
        steps = [([("p", tokens["p"][:70], list(range(70))), ("q", tokens["q"][:1], [0])], []),
                 ([("p", tokens["p"][70:71], [0]), ("q", tokens["q"][1:19], list(range(18)))], [])]
        steps += [([("p", [tokens["p"][i]], [0])] + ([("q", [tokens["q"][19]], [0])] if i == 71 else []), []) for i in range(71, 100)]
        tm.check(tokens, harness.replay(tm.runner(16), steps), f"heads {heads}/{kv_heads} of {dim}, {vdim}")


@pytest.mark.parametrize("width", [50, 70])
def test_widths_that_are_no_multiple_of_four(width):
    """No 16-byte rows anywhere: every kernel's element-by-element form, in both dtypes."""
    cfg = {"architecture": "Bunosun", "vocab": 67, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
           "layers": [bt.attention_layer(2, 1, 10, 14, 11, 6, bt.moe(6, 2, 22, 3, 2, 18), diff=0.3, factor=2.0),
                      bt.delta_layer(2, 1, 10, 14, 3, bt.moe(6, 2, 22, 3, 2, 18))],
           "loop": {"start": 0, "stop": 2, "times": 2}}
    for dtype in ("float32", "bfloat16"):
        tm = bt.TinyBunosun("-", dtype, cfg=cfg, seed=2)
        tokens = {"p": bt.random_tokens(cfg, 90, 70)}
        steps = [([("p", tokens["p"][:60], list(range(60)))], [])]
        steps += [([("p", [t], [0])], []) for t in tokens["p"][60:]]
        tm.check(tokens, harness.replay(tm.runner(8), steps), f"width {width}")


def test_missing_and_misshapen_tensors_are_named():
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.weights.loader import WeightsError

    cfg, _ = bt.CONFIGS["B"]
    weights = bt.random_weights(cfg, 1)
    del weights["l1.mix.lq2"]
    weights["l0.mix.a2"] = weights["l0.mix.a2"][:-1].contiguous()
    tm = bt.TinyBunosun("B", "float32", weights=weights)
    with pytest.raises((WeightsError, ValueError)) as error:
        load_model(tm.folder, "float32", DEV)
    assert "l1.mix.lq2" in str(error.value) and "l0.mix.a2" in str(error.value)


# --------------------------------------------------------------------------- the engine
def _plain_greedy(tm, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(tm.plain_logits(tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_greedy_generation_through_the_engine(cuda_graphs):
    """Requests of unequal lengths through Engine.submit / step: admission, prompt portions of 16
    tokens beside decoding requests, more requests than slots (so slots and pages are used again),
    eager and captured decode steps; float32 tokens equal the plain implementation's."""
    from pulsarlm_b200.engine.engine import Engine

    tm = _model("A", "float32")
    engine = Engine(tm.folder, dtype="float32", device=DEV, page_size=16, n_pages=40, max_requests=3,
                    prefill_tokens_per_step=16, cuda_graphs=cuda_graphs)
    prompts = [bt.random_tokens(tm.cfg, n, 60 + i) for i, n in enumerate([40, 3, 21, 9, 30])]
    requests = [engine.submit(p, max_tokens=12, ignore_eos=True) for p in prompts]
    for _ in range(400):
        if not engine.has_work():
            break
        engine.step()
    assert not engine.has_work()
    for prompt, request in zip(prompts, requests):
        assert list(request.output) == _plain_greedy(tm, prompt, 12)
    if cuda_graphs:
        assert engine.runner.graph_steps > 0


def test_many_requests_decode_in_captured_steps_through_the_grouped_experts():
    """Sixty requests at once in bfloat16: their decode steps are long enough for the experts' sorted
    path, inside captured steps; every request ends with as many tokens as asked."""
    from pulsarlm_b200.engine.engine import Engine

    tm = _model("A", "bfloat16")
    engine = Engine(tm.folder, dtype="bfloat16", device=DEV, page_size=16, n_pages=200, max_requests=60,
                    prefill_tokens_per_step=256, cuda_graphs=True)
    prompts = [bt.random_tokens(tm.cfg, 3 + i % 4, 200 + i) for i in range(60)]
    requests = [engine.submit(p, max_tokens=6, ignore_eos=True) for p in prompts]
    for _ in range(400):
        if not engine.has_work():
            break
        engine.step()
    assert not engine.has_work() and engine.runner.graph_steps > 0
    assert all(len(r.output) == 6 and r.finish_reason == "length" for r in requests)


def test_engine_preempts_and_recomputes_with_states():
    """So few pages that running requests are preempted (pages and state slots given back, the
    request recomputed from its start later): the tokens are still the plain implementation's, so
    no state of an earlier life leaks into the recomputation."""
    from pulsarlm_b200.engine.engine import Engine

    cfg = json.loads(json.dumps(bt.CONFIGS["B"][0]))  # (its first attention layer has no window: every page is kept)
    tm = bt.TinyBunosun("-", "float32", seed=4, cfg=cfg)
    engine = Engine(tm.folder, dtype="float32", device=DEV, page_size=16, n_pages=7, max_requests=4,
                    prefill_tokens_per_step=16)
    prompts = [bt.random_tokens(cfg, n, 95 + i) for i, n in enumerate([30, 25, 20])]
    requests = [engine.submit(p, max_tokens=20, ignore_eos=True) for p in prompts]
    for _ in range(600):
        if not engine.has_work():
            break
        engine.step()
    assert not engine.has_work() and engine.scheduler.preemptions > 0
    for prompt, request in zip(prompts, requests):
        assert request.finish_reason == "length"
        assert list(request.output) == _plain_greedy(tm, prompt, 20)


def test_engine_in_bfloat16_with_captured_steps_stays_close():
    from pulsarlm_b200.engine.engine import Engine

    tm = _model("C", "bfloat16")
    engine = Engine(tm.folder, dtype="bfloat16", device=DEV, page_size=16, n_pages=40, max_requests=4,
                    prefill_tokens_per_step=32, record_logits=True)
    prompts = [bt.random_tokens(tm.cfg, n, 70 + i) for i, n in enumerate([50, 7, 33])]
    requests = [engine.submit(p, max_tokens=20, ignore_eos=True) for p in prompts]
    while engine.has_work():
        engine.step()
    errors = []
    for prompt, request in zip(prompts, requests):
        full = list(prompt) + list(request.output)
        ref = tm.plain_logits(full[:-1])
        errors += [bt.relative_error(row, ref[len(prompt) - 1 + i]) for i, row in enumerate(request.logits)]
    errors.sort()
    assert errors[len(errors) * 9 // 10] < bt.TOLERANCE["bfloat16"] and errors[-1] < 0.5


def test_command_line_random_model_generate_and_replay(tmp_path, capsys):
    """`models list`, `models random`, `generate` and `replay` of the command line for this
    architecture: greedy tokens equal the plain implementation's on the written weights, and the
    replayed logits too."""
    import io

    import numpy as np
    from safetensors.torch import load_file

    from pulsarlm_b200 import cli
    from pulsarlm_b200.engine import trace

    assert cli.main(["models", "list"]) == 0
    assert "Bunosun" in capsys.readouterr().out.split()
    cfg = json.loads(json.dumps(bt.CONFIGS["A"][0]))
    for layer in cfg["layers"]:
        if layer["type"] == "channel_delta":
            layer["mixer"]["decay_rank"] = 5
            layer["mixer"]["gate_rank"] = 7
    folder = str(tmp_path / "model")
    with open(tmp_path / "c.json", "w") as f:
        json.dump(cfg, f)
    assert cli.main(["models", "random", folder, "--config", str(tmp_path / "c.json"), "--seed", "3",
                     "--dtype", "float32", "--std", "0.3"]) == 0
    capsys.readouterr()
    weights = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    prompt = bt.random_tokens(cfg, 19, 90)
    assert cli.main(["generate", folder, "--dtype", "float32", "--prompt_ids", ",".join(map(str, prompt)),
                     "--max_tokens", "8", "--ignore_eos"]) == 0
    record = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    tokens = list(prompt)
    for _ in range(8):
        tokens.append(int(plain.forward(cfg, weights, tokens)[0][-1].argmax()))
    assert record["output_ids"] == tokens[len(prompt):]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:11], "want": [3, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[11:12], "want": [0]}], "end": ["a"]}]
    out = io.StringIO()
    assert trace.run(["--model", folder, "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "64"],
                     stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out) == 0
    assert out.getvalue().split() == ["done", "0", "done", "1"]
    ref = plain.forward(cfg, weights, tokens[:12])[0]
    got0 = torch.from_numpy(np.fromfile(str(tmp_path / "out" / "0.f32"), dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(str(tmp_path / "out" / "1.f32"), dtype="<f4").reshape(1, -1))
    assert bt.relative_error(got0, ref[[3, 10]]) < 2e-4 and bt.relative_error(got1, ref[[11]]) < 2e-4
