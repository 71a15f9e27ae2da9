"""Differential attention as a mixer part: every head has two softmax maps over the same values and puts out
their weighted difference,

    o = a1 - lambda a2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      (one number per layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)                                (per head, no weight)

The q projection has heads x 2 x dim rows and the k projection kv_heads x 2 x dim, head by head as
[map 1, map 2]; both maps of a head read the value head of its group.  This is grouped-query attention with
twice the heads and with values that two key heads share, so the part is `GQAAttention` with
`value_heads = kv_heads`, a 32-bit output, and one more kernel that combines the maps.  The rows of W_q are
reordered once at load time so that the query heads of one key head (a group's map) lie side by side.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..config.plan import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from .attention import GQAAttention
from .base import register_part

LAMBDA_NAMES = {"lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}


class DifferentialAttention(GQAAttention):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 diff: float, eps: float, window: Optional[int] = None, prefix: str = "", names: Optional[dict] = None):
        super().__init__(hidden_size, 2 * num_heads, 2 * num_kv_heads, head_dim, scale,
                         qk_norm=PartSpec("rms_norm", {"size": head_dim, "eps": eps}), window=window, prefix=prefix,
                         value_dim=value_dim, names=dict(LAMBDA_NAMES, **(names or {})), value_heads=num_kv_heads,
                         out_float32=True)
        self.heads, self.kv_heads, self.diff, self.eps = int(num_heads), int(num_kv_heads), float(diff), float(eps)
        self.lam = None

    def output_width(self) -> int:
        return self.heads * self.value_dim

    def weight_specs(self, prefix: str) -> dict:
        specs = super().weight_specs(prefix)
        p = prefix + self.prefix
        specs.update({p + self.names[k]: WeightSpec((self.head_dim,), "bias") for k in LAMBDA_NAMES})
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        super().bind(weights, prefix, dtype, device)
        p = prefix + self.prefix
        vectors = {k: weights[p + self.names[k]] for k in LAMBDA_NAMES}
        getattr(weights, "wait", lambda: None)()              # a streamed checkpoint: the tensors are in place now
        lq1, lk1, lq2, lk2 = (vectors[k].double().cpu() for k in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff
        # query heads as the kernels group them: [kv head, map, head in group] instead of [head, map]
        H, G, d = self.heads, self.kv_heads, self.head_dim
        r = H // G
        order = torch.arange(2 * H, device=self.w_qkv.device).view(G, r, 2).permute(0, 2, 1).reshape(-1)
        rows = (order[:, None] * d + torch.arange(d, device=self.w_qkv.device)[None, :]).reshape(-1)
        self.w_qkv[:rows.numel()] = self.w_qkv[:rows.numel()][rows]

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        from .linear import linear
        N = ctx.n_tokens
        maps = self.mix(x, ctx, cache)                       # [N, kv head, map, head in group, vdim] float32
        combined = ctx.scratch.get("attn.combined", (N, self.heads * self.value_dim), ctx.dtype)
        ops.diff_combine(maps, combined, N, self.heads, self.heads // self.kv_heads, self.value_dim, self.lam, self.eps,
                         1.0 - self.diff)
        out = ctx.scratch.get("mixer.out", (N, self.hidden_size), ctx.dtype)
        return linear(combined, self.w_o, out)


register_part("mixer", "differential_attention", DifferentialAttention)
