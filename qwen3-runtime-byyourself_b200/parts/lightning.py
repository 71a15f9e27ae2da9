"""Linear attention with a per-head decay ("lightning" attention) as a mixer part.

q, k, v = SiLU of their projections (heads x dim, heads x dim, heads x vdim); per head a state S [dim, vdim]
that lives in float32 in the cache's state rows (zero for a new sequence, carried from step to step):

    S_t = decay_h S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t      (no other scale)

The heads of a token, side by side, are brought to unit rms together, multiplied by a weight and by
sigmoid(W_g x), and projected by W_o.  The four input projections run as one product; the recurrence, the
activation and everything that enters them are 32-bit whatever the compute type.  It needs no keys in the
cache: `CacheNeed("none", state_shape=(heads, dim, vdim))`.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache.book import CacheNeed
from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .base import Part, register_part
from .linear import linear

TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
chunk_rows = 16      # from this many new tokens of the longest sequence on, the chunked form runs


class LightningAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float], eps: float,
                 prefix: str = "", names: Optional[dict] = None):
        if len(decay) != num_heads:
            raise ValueError("one decay per head")
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError("head sizes up to 256")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.decay_values, self.eps, self.prefix = [float(v) for v in decay], float(eps), prefix
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.w_in = self.w_o = self.norm_weight = self.decay = None

    def weight_specs(self, prefix: str) -> dict:
        p, n, H = prefix + self.prefix, self.names, self.hidden_size
        qk, vg = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        return {p + n["q"]: WeightSpec((qk, H)), p + n["k"]: WeightSpec((qk, H)), p + n["v"]: WeightSpec((vg, H)),
                p + n["g"]: WeightSpec((vg, H)), p + n["o"]: WeightSpec((H, vg)), p + n["norm"]: WeightSpec((vg,), "norm")}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in = fuse_rows(weights, [p + n[k] for k in ("q", "k", "v", "g")])
        self.w_o = weights.pop(p + n["o"]).contiguous()
        self.norm_weight = weights[p + n["norm"]].to(device=device, dtype=torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def cache_need(self) -> CacheNeed:
        return CacheNeed("none", state_shape=(self.num_heads, self.head_dim, self.value_dim))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, h, d, vd = ctx.n_tokens, self.num_heads, self.head_dim, self.value_dim
        proj = ctx.scratch.get("lightning.proj", (N, 2 * h * (d + vd)), ctx.dtype)
        linear(x, self.w_in, proj)
        o = ctx.scratch.get("lightning.o", (N, h * vd), torch.float32)
        chunked = not ctx.is_decode and ctx.max_new >= chunk_rows and ops.lightning_chunks_fit(d, vd)
        ops.lightning_attention(proj, cache.state, self.decay, ctx.seq_start, ctx.seq_slots, o, ctx.n_seqs, h, d, vd, chunked)
        gated = ctx.scratch.get("lightning.gated", (N, h * vd), ctx.dtype)
        ops.gated_norm(o, proj[:, 2 * h * d + h * vd:], self.norm_weight, self.eps, gated)
        out = ctx.scratch.get("mixer.out", (N, self.hidden_size), ctx.dtype)
        return linear(gated, self.w_o, out)


register_part("mixer", "lightning_attention", LightningAttention)
