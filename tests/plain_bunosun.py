"""A plain, slow implementation of the Bunosun decoder in float64 torch on the CPU, one
function per mechanism, written from the architecture's equations. It shares no code
with the engine: whole sequences at once, no cache, no pages, no state slots.

Notation: x [T, W] the residual stream, h a sublayer's input, weights by their
checkpoint names ([out, in], applied as W h).
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the scale minus one."""
    return rms(x, eps) * (1.0 + weight)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float) -> torch.Tensor:
    """x [T, ..., D]: columns (2i, 2i + 1), i < dims / 2, turn by positions * base^(-2i / dims) / factor."""
    if dims == 0:
        return x
    out = x.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    angle = positions.double()[:, None] * (base ** (-2.0 * i / dims) / factor)[None]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = angle.cos().view(shape), angle.sin().view(shape)
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


def visible(n: int, window: int | None) -> torch.Tensor:
    """[query, key] True where key <= query and, with a window, query - key < window."""
    i = torch.arange(n)
    back = i[:, None] - i[None, :]
    return (back >= 0) & (back < window if window else back >= 0)


def differential_attention(mixer: dict, w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    q = (h @ w[p + "q"].T).view(n, heads, 2, dim)
    k = (h @ w[p + "k"].T).view(n, kv_heads, 2, dim)
    v = (h @ w[p + "v"].T).view(n, kv_heads, vdim)
    rot = mixer.get("rot")
    if rot:
        positions = torch.arange(n)
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_pairs(k, positions, rot["dims"], rot["base"], factor)
    see = visible(n, (mixer.get("mask") or {}).get("size"))
    lam = (math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum()))
           + mixer["diff"])
    out = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for head in range(heads):
        g = head // (heads // kv_heads)
        maps = []
        for m in range(2):
            scores = (q[:, head, m] @ k[:, g, m].T) * mixer["scale"]
            maps.append(torch.softmax(scores.masked_fill(~see, float("-inf")), dim=-1) @ v[:, g])
        out[:, head] = rms(maps[0] - lam * maps[1], eps) * (1.0 - mixer["diff"])
    return out.reshape(n, heads * vdim) @ w[p + "o"].T


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y[t] = sum_j taps[:, j] * x[t - (K - 1) + j], zeros before the start; then silu."""
    n, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = sum(padded[j:j + n] * taps[:, j] for j in range(k))
    return y * torch.sigmoid(y)


def channel_delta(mixer: dict, w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    heads, qk_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    q = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(n, qk_heads, dim)
    k = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(n, qk_heads, dim)
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(n, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    step = torch.nn.functional.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(n, heads, dim)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(n, heads, vdim)
    out = delta_scan(q, k, v, beta, decay)
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(n, heads * vdim) @ w[p + "o"].T


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """The recurrence alone. q, k [T, qk_heads, dim] (already unit vectors), v [T, heads, vdim], beta
    [T, heads], decay [T, heads, dim]; the state starts at zero. Returns o [T, heads, vdim]."""
    n, heads, vdim = v.shape
    qk_heads, dim = q.shape[1], q.shape[2]
    state = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    out = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for t in range(n):
        for head in range(heads):
            g = head // (heads // qk_heads)
            s = decay[t, head][:, None] * state[head]
            u = beta[t, head] * (v[t, head] - s.T @ k[t, g])
            s = s + torch.outer(k[t, g], u)
            out[t, head] = s.T @ q[t, g]
            state[head] = s
    return out


def gated_expert(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    z = h @ w[p + "gate"].T
    return (z * torch.sigmoid(z) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(mlp: dict, w: dict, p: str, h: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top])."""
    router = mlp["router"]
    experts, top = router["experts"], router["top"]
    groups = router.get("groups") or {}
    count = groups.get("count", 1)
    keep = groups.get("keep", count)
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = scores + w[p + "correction"]
    n = h.shape[0]
    chosen = torch.zeros(n, top, dtype=torch.long)
    for t in range(n):
        per = experts // count
        best = sorted(range(count), key=lambda g: (-float(choice[t, g * per:(g + 1) * per].max()), g))[:keep]
        open_ = [e for e in range(experts) if e // per in best]
        open_.sort(key=lambda e: (-float(choice[t, e]), e))
        chosen[t] = torch.tensor(open_[:top])
    weights = scores.gather(1, chosen)
    return chosen, weights / (weights.sum(-1, keepdim=True) + 1e-20)


def routed_experts(mlp: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    chosen, weights = route(mlp, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(chosen.shape[1]):
            out[t] += weights[t, j] * gated_expert(w, f"{p}e{int(chosen[t, j])}.", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + gated_expert(w, p + "shared.", h)
    return out


def run_order(cfg: dict) -> tuple[list[int], set[int]]:
    """(layers in the order they run, places in that order where a later pass of the loop begins)."""
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = list(range(loop["start"]))
    again = set()
    for time in range(loop["times"]):
        if time > 0 and loop["stop"] > loop["start"]:
            again.add(len(order))
        order += list(range(loop["start"], loop["stop"]))
    return order + list(range(loop["stop"], len(cfg["layers"]))), again


def forward(cfg: dict, w: dict, tokens: list[int]) -> tuple[torch.Tensor, list[torch.Tensor]]:
    """(logits [T, vocab], the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    entered = x.clone()
    order, again = run_order(cfg)
    streams = []
    for run, i in enumerate(order):
        if run in again:
            x = x + entered
        layer, p = cfg["layers"][i], f"l{i}."
        h1 = offset_norm(x, w[p + "norm1"], eps)
        mix = (differential_attention if layer["type"] == "attention" else channel_delta)(
            layer["mixer"], w, p + "mix.", h1, eps)
        update = mix * w[p + "ls1"]
        if layer.get("mlp"):
            update = update + routed_experts(layer["mlp"], w, p + "mlp.", offset_norm(x, w[p + "norm2"], eps)) * w[p + "ls2"]
        x = x + update
        streams.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T, streams
