"""A plain, slow restatement of the Rerilorn decoder in torch on the CPU: one function
per mechanism, written from the equations and sharing nothing with the package's parts
or kernels. Everything runs in the dtype of the tensors it is given (float64 in the
tests). A sequence's state between calls is a plain dict, so a prompt can be fed whole,
in portions or token by token.

Notation: x [T, W] is the residual stream of one sequence, h a sublayer's input.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps), times `weight` when given; over the last axis."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def short_convolution(h: torch.Tensor, weight: torch.Tensor, history: torch.Tensor | None):
    """h [T, W], weight [W, taps]: returns (h + c, new history) with
    c[t] = sum_j weight[:, j] * h[t - (taps - 1) + j], rows before the sequence's start
    being zero. `history` [taps - 1, W] holds the inputs of the tokens just before."""
    taps = weight.shape[1]
    width = h.shape[1]
    if history is None:
        history = torch.zeros((taps - 1, width), dtype=h.dtype)
    padded = torch.cat([history, h], dim=0)
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] += weight[:, j] * padded[t + j]
    return out, padded[padded.shape[0] - (taps - 1):].clone()


def delta_rule_scan(r, k, v, decay, removal, state):
    """One head. r, k, decay, removal [T, K]; v [T, V]; state [K, V] (changed in place).
    S <- diag(decay) S - (removal * u) (u^T S) + k v^T with u = k / sqrt(|k|^2 + 1e-6),
    both products reading the state as it was before the token; o = S^T r."""
    out = []
    for t in range(r.shape[0]):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum() + 1e-6)
        old = state.clone()
        state.copy_(decay[t][:, None] * old - torch.outer(removal[t] * u, u @ old) + torch.outer(k[t], v[t]))
        out.append(state.t() @ r[t])
    return torch.stack(out)


def general_delta_mixer(h, w: dict, heads: int, dim: int, eps: float, state: torch.Tensor | None):
    """h [T, W]; w: the layer's mixer tensors by their short names; state [heads, dim, dim]."""
    T = h.shape[0]
    if state is None:
        state = torch.zeros((heads, dim, dim), dtype=h.dtype)
    r = (h @ w["r"].t()).view(T, heads, dim)
    k = (h @ w["k"].t()).view(T, heads, dim)
    v = (h @ w["v"].t()).view(T, heads, dim)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w["w1"].t()) @ w["w2"].t() + w["w0"]))
    removal = torch.sigmoid(h @ w["a"].t() + w["a.b"])
    decay, removal = decay.view(T, heads, dim), removal.view(T, heads, dim)
    o = torch.stack([delta_rule_scan(r[:, i], k[:, i], v[:, i], decay[:, i], removal[:, i], state[i])
                     for i in range(heads)], dim=1)                       # [T, heads, dim]
    o = rms_norm(o, None, eps).reshape(T, heads * dim) * w["norm"]
    o = o * torch.sigmoid(h @ w["g"].t())
    return o @ w["o"].t(), state


def latent_attention_mixer(h, w: dict, heads: int, dim: int, vdim: int, scale: float, window: int, eps: float,
                           latents: torch.Tensor | None):
    """h [T, W]; `latents` [P, rank] are the cached latents of the P tokens before. Query i
    (absolute position P + i) sees key j when 0 <= i_abs - j < window. The softmax's
    denominator holds one more term exp(sink) per head."""
    T = h.shape[0]
    q = (h @ w["q"].t()).view(T, heads, dim)
    c = rms_norm(h @ w["dkv"].t(), w["dkv.norm"], eps)
    allc = c if latents is None else torch.cat([latents, c], dim=0)
    past = allc.shape[0] - T
    keys = (allc @ w["uk"].t()).view(-1, heads, dim)
    values = (allc @ w["uv"].t()).view(-1, heads, vdim)
    gate = torch.sigmoid(h @ w["g"].t())                                  # [T, heads]
    out = torch.zeros((T, heads, vdim), dtype=h.dtype)
    for i in range(T):
        at = past + i
        lo = max(0, at - window + 1)
        for head in range(heads):
            s = (keys[lo:at + 1, head] @ q[i, head]) * scale
            m = torch.maximum(s.max(), w["sink"][head])
            e = torch.exp(s - m)
            denom = e.sum() + torch.exp(w["sink"][head] - m)
            out[i, head] = (e / denom) @ values[lo:at + 1, head] * gate[i, head]
    return out.reshape(T, heads * vdim) @ w["o"].t(), allc


def dense_feed_forward(h, w: dict):
    z = torch.relu(h @ w["up"].t() + w["up.b"])
    return (z * z) @ w["down"].t() + w["down.b"]


def _sub(tensors: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], state: dict | None = None,
            layer_outputs: list | None = None):
    """Runs `tokens` after what `state` holds; returns (logits [T, vocab], state)."""
    state = {} if state is None else state
    eps = float(config["norm"]["eps"])
    mult = float(config["residual_mult"])
    x = tensors["embed"][torch.tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, tensors[p + "norm1"], eps)
        if config.get("canon"):
            h, state[p + "canon1"] = short_convolution(h, tensors[p + "canon1"], state.get(p + "canon1"))
        mix = _sub(tensors, p + "mix.")
        if layer["type"] == "general_delta":
            y, state[p + "S"] = general_delta_mixer(h, mix, int(m["heads"]), int(m["dim"]), eps, state.get(p + "S"))
        elif layer["type"] == "latent_attention":
            y, state[p + "c"] = latent_attention_mixer(h, mix, int(m["heads"]), int(m["dim"]), int(m["vdim"]),
                                                       float(m["scale"]), int(m["mask"]["size"]) if m.get("mask") else 1 << 30, eps,
                                                       state.get(p + "c"))
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(y, tensors[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[p + "norm2"], eps)
            if config.get("canon"):
                h, state[p + "canon2"] = short_convolution(h, tensors[p + "canon2"], state.get(p + "canon2"))
            y = dense_feed_forward(h, _sub(tensors, p + "mlp."))
            x = x + mult * rms_norm(y, tensors[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    h = rms_norm(x, tensors["final.norm"], eps)
    return h @ tensors["embed"].t(), state
