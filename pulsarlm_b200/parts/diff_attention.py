"""Differential attention: every head forms two softmax maps over the same values and
outputs their difference, normed per head."""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from .attention import Attention
from .linear import linear
from .registry import BuildContext, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed

MAPS = 2


@register_part("mixer", "diff_attention")
class DiffAttention(Attention):
    """q = Wq h [heads, 2, dim], k = Wk h [kv_heads, 2, dim], v = Wv h [kv_heads, vdim]; map m of
    head h is causal softmax attention of q[h, m] over k[g, m] (g = h // (heads / kv_heads))
    with the values v[g]; then

        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff          (one number for the layer)
        o_h = a_h1 - lambda * a_h2;  out_h = (1 - diff) * o_h / sqrt(mean(o_h^2) + eps)

    and the o projection over the concatenated heads. The position encoding (a "position"
    PartSpec; "rope_pairs" rotates neighbouring pairs) is applied within every map.

    The maps run on the ordinary paged attention kernels as 2 * heads query heads over
    kv_heads kv heads of a common row size Dp = max(2 * dim, vdim) (rounded up to what the
    tensor-core kernels take where that is near): map m's query occupies columns [m * dim,
    (m + 1) * dim) of a zero row, the cached key row is [k_1 | k_2 | 0], the value row [v | 0]
    (csrc/rope_maps.cu). Everything the base class knows (window, split counts, work lists,
    prompt tiles, captured steps) applies unchanged; the maps' outputs are combined by one
    small kernel (fp32).

    params: hidden_size, n_heads, n_kv_heads, head_dim (of one map), value_dim, diff, eps,
    scale (optional), window (optional), position. tensors: q [nh*2*hd, H], k [nkv*2*hd, H],
    v [nkv*vd, H], o [H, nh*vd], lq1, lk1, lq2, lk2 [hd]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        p = spec.params
        self.true_heads = int(p["n_heads"])
        self.map_dim = int(p["head_dim"])
        self.value_dim = int(p["value_dim"])
        self.diff = float(p["diff"])
        self.eps = float(p["eps"])
        self.padded = padded_row(self.map_dim, self.value_dim)
        scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.map_dim)
        inner = PartSpec(spec.kind, {**p, "n_heads": MAPS * self.true_heads, "head_dim": self.padded, "scale": scale},
                         spec.tensors)
        super().__init__(inner, ctx)
        self.spec = spec
        if p.get("cache_from") is not None or p.get("softcap") or p.get("qk_norm_eps"):
            raise ValueError("diff_attention: cache_from, softcap and q/k norms are not supported")
        self.lam: float | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, nkv, hd, vd = (int(p[k]) for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim", "value_dim"))
        needs = {t["q"]: TensorNeed((nh * MAPS * hd, h)), t["k"]: TensorNeed((nkv * MAPS * hd, h)),
                 t["v"]: TensorNeed((nkv * vd, h)), t["o"]: TensorNeed((h, nh * vd))}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            needs[t[name]] = TensorNeed((hd,), role="offset")
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.qkv = torch.cat([tensors[t["q"]], tensors[t["k"]], tensors[t["v"]]], dim=0).contiguous()
        self.o = tensors[t["o"]].contiguous()
        lq1, lk1, lq2, lk2 = (tensors[t[name]].float() for name in ("lq1", "lk1", "lq2", "lk2"))
        # (a constant of the weights: formed once, in fp32)
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())) + self.diff

    def cache_need(self) -> KVCacheNeed:
        return KVCacheNeed(self.n_kv, self.padded, self.window, self.n_heads)

    def _folds_rope(self, tokens, batch, inv_freq, rotary) -> bool:
        return False  # (the maps' layout and rotation are a kernel of their own)

    def native_choice(self, tokens, batch, row_stride):
        return None

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, nkv, hd, vd = self.true_heads, self.n_kv, self.map_dim, self.value_dim
        cache = self.cache
        table = batch.tables[cache.group]
        qkv = linear(h, self.qkv)
        q_end, k_end = nh * MAPS * hd, (nh + nkv) * MAPS * hd
        q = torch.empty((tokens, MAPS * nh, self.padded), dtype=h.dtype, device=h.device)
        inv_freq, rotary = self.position.table()
        ops.rope_maps_write(qkv[:, :q_end], qkv[:, q_end:k_end], qkv[:, k_end:], batch.pos, batch.entry, table,
                            cache.k_pool, cache.v_pool, cache.page_size, inv_freq, rotary, nh, nkv, MAPS, hd, vd, q,
                            batch.status)
        maps = torch.empty_like(q)
        self.attend(q, maps, table, batch)
        out = torch.empty((tokens, nh * vd), dtype=h.dtype, device=h.device)
        ops.diff_combine(maps, out, nh, vd, self.lam, self.eps, 1.0 - self.diff)
        return linear(out, self.o)


def padded_row(map_dim: int, value_dim: int) -> int:
    """The common row size of queries, keys and values: at least both maps' keys and the
    values, rounded up to a multiple of 16 (the tensor-core kernels' step) and, from 48 up to
    128, to 64 or 128 where that is within a third (the sizes the tcgen05 prompt kernel takes)."""
    need = max(MAPS * map_dim, value_dim)
    row = -(-need // 16) * 16
    for size in (64, 128):
        if row <= size and 4 * need >= 3 * size:
            return size
    return row
