"""Attention over a cached low-rank latent: one row per token serves every head as key and value."""

from __future__ import annotations

import torch

from ..kernels import ops
from .attention import KVBinding
from .linear import linear
from .registry import BuildContext, Part, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed


def per_head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, h, :] = x[:, h, :] @ weight[h]^T for x [T, H, K], weight [H, N, K], out [T, H, N]
    (a view whose last axis is contiguous). bfloat16: one batched library product that
    writes the strided output in place; float32: the package's own fp32 product per head."""
    heads = x.shape[1]
    if x.dtype == torch.float32:
        for h in range(heads):
            ops.gemm_f32(x[:, h], weight[h], out[:, h])
        return
    torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """Causal attention whose keys and values are projections of a shared latent:

        q = Wq h                       [heads, dim]
        c = rmsnorm(Wd h) * n          [rank]: the only thing cached per token
        k_h = Wuk_h c, v_h = Wuv_h c   per head
        p = softmax over {(q_h . k_h) * scale of the keys in reach} and one sink term exp(s_h)
        out = Wo concat_h(sigmoid(Wg h)_h * sum_j p_j v_h,j)

    Keys and values are never formed: with q'_h = Wuk_h^T q_h the scores are q'_h . c_j, and
    the weighted sum of the latents goes through Wuv_h afterwards, so attention runs over
    the paged latents with one shared "kv head" of size rank. No position encoding.

    params: hidden_size, n_heads, head_dim (of q and k), value_dim, latent_rank, scale,
    window (None: every earlier token; n: the token itself and the n - 1 before it),
    eps (of the latent's norm), sink (whether the softmax has the sink term), gate
    (whether heads are gated). tensors: q [nh*hd, H], down [rank, H], latent_norm [rank],
    up_k [nh*hd, rank], up_v [nh*vd, rank], sink [nh], gate [nh, H], o [H, nh*vd]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.value_dim = int(self.param("value_dim"))
        self.rank = int(self.param("latent_rank"))
        self.scale = float(self.param("scale"))
        self.window = int(p["window"]) if p.get("window") else None
        self.eps = float(self.param("eps"))
        self.has_sink = bool(p.get("sink", False))
        self.has_gate = bool(p.get("gate", False))
        self.stacked: torch.Tensor | None = None
        self.up_k = self.up_v = self.o = self.latent_norm = self.sink = None
        self.cache: KVBinding | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, hd, vd, rank = (int(p[k]) for k in ("hidden_size", "n_heads", "head_dim", "value_dim", "latent_rank"))
        needs = {t["q"]: TensorNeed((nh * hd, h)), t["down"]: TensorNeed((rank, h)),
                 t["latent_norm"]: TensorNeed((rank,), role="vector"), t["up_k"]: TensorNeed((nh * hd, rank)),
                 t["up_v"]: TensorNeed((nh * vd, rank)), t["o"]: TensorNeed((h, nh * vd))}
        if p.get("sink"):
            needs[t["sink"]] = TensorNeed((nh,), role="offset")
        if p.get("gate"):
            needs[t["gate"]] = TensorNeed((nh, h))
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        nh, hd, vd, rank = self.n_heads, self.head_dim, self.value_dim, self.rank
        parts = [tensors[t["q"]], tensors[t["down"]]] + ([tensors[t["gate"]]] if self.has_gate else [])
        self.stacked = torch.cat(parts, dim=0).contiguous()      # q, latent, gate logits from one product
        # q'_h = Wuk_h^T q_h as a product with rows [rank] over dim: the transposed blocks.
        self.up_k = tensors[t["up_k"]].view(nh, hd, rank).transpose(1, 2).contiguous()   # [nh, rank, hd]
        self.up_v = tensors[t["up_v"]].view(nh, vd, rank).contiguous()                   # [nh, vd, rank]
        self.o = tensors[t["o"]].contiguous()
        self.latent_norm = tensors[t["latent_norm"]].float().contiguous()
        self.sink = tensors[t["sink"]].float().contiguous() if self.has_sink else None

    def cache_need(self) -> KVCacheNeed:
        return KVCacheNeed(1, self.rank, self.window, self.n_heads, planes=1)

    def bind_cache(self, binding: KVBinding) -> None:
        self.cache = binding

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, hd, vd, rank = self.n_heads, self.head_dim, self.value_dim, self.rank
        cache = self.cache
        table = batch.tables[cache.group]
        proj = linear(h, self.stacked)
        q = proj[:, : nh * hd].view(tokens, nh, hd)
        ops.norm_write_paged(proj[:, nh * hd: nh * hd + rank], self.latent_norm, self.eps, batch.pos, batch.entry,
                             table, cache.k_pool, cache.page_size, batch.status)
        gate = proj[:, nh * hd + rank:] if self.has_gate else None
        q_latent = torch.empty((tokens, nh, rank), dtype=h.dtype, device=h.device)
        per_head_linear(q, self.up_k, q_latent)
        mixed = torch.empty((tokens, nh, rank), dtype=h.dtype, device=h.device)
        self.attend(q_latent, mixed, table, batch, gate)
        out = torch.empty((tokens, nh, vd), dtype=h.dtype, device=h.device)
        per_head_linear(mixed, self.up_v, out)
        return linear(out.view(tokens, nh * vd), self.o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, table: torch.Tensor, batch, gate) -> None:
        """out[t, h] = gate * sum_j p_j c_j over the latents in reach of token t."""
        cache = self.cache
        ops.attention_simt(q, cache.k_pool, cache.v_pool, table, batch.pos, batch.entry, out, cache.page_size,
                           self.window, self.scale, batch.status, sinks=self.sink, gate=gate)
