"""Steps between layers that rewrite the hidden state from itself and the embedding's output.

`mix_in`: x <- W [x; x0] with W [hidden, 2 hidden], x first: the state and the embedding output
x0 are laid side by side (rounded to the compute type, as every input of a product) and one
product gives the new state, in float32.  A model that runs a stretch of layers several times
uses it at the start of every pass, so that the input is fed in again each time.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .block import settle
from .linear import linear


class MixIn(Part):
    def __init__(self, hidden_size: int):
        self.hidden_size = int(hidden_size)
        self.weight = None
        self._turn = 0

    def weight_specs(self, name: str) -> dict:
        return {name: WeightSpec((self.hidden_size, 2 * self.hidden_size))}

    def bind(self, weights: dict, name: str, dtype, device) -> None:
        self.weight = weights[name].contiguous()

    def forward(self, residual, delta, x0, ctx):
        """(residual, delta) -> (W [residual + delta; x0], None); the result lies in a buffer of its own, `x0` and the
        buffer of `residual` are left as they are (apart from the pending sum, which is done in place)."""
        if residual.dtype != torch.float32:
            raise ops.KernelError("mix_in works on a float32 hidden state")
        N, H = residual.shape
        settle(residual, delta)
        both = ctx.scratch.get("stream.both", (N, 2 * H), ctx.dtype)
        ops.concat_cast(residual, x0, both)
        # two buffers take turns, so that the input of a step is never its output
        names = ("stream.mixed_a", "stream.mixed_b")
        out = ctx.scratch.get(names[0], (N, H), torch.float32)
        if out.data_ptr() == residual.data_ptr():
            out = ctx.scratch.get(names[1], (N, H), torch.float32)
        linear(both, self.weight, out)
        return out, None


register_part("stream", "mix_in", MixIn)
