"""The arrangements of a layer.

`pre_norm`: x += mixer(norm(x)); x += feed_forward(norm(x))  (src/model/decoder_layer.cpp:63-98).
The hidden state travels as (residual, delta): each sum is done by the next norm's
kernel, which writes the new residual and its normalised copy in one pass.

`sandwich_norm`: a norm before and a norm after every sublayer, x += norm_b(mixer(norm_a(x))),
then the same around the feed-forward (which a layer may lack), on a hidden state that is kept
in float32 whatever the compute type.  Here `delta` is a `NormedBranch`: a sublayer's output
that still has to be normalised and added.  Whoever comes next does it (the next block, a
stream step or the model's tail), in the same kernel that normalises the sum for its own
input, so a layer costs two passes over the hidden state.
"""
from __future__ import annotations

from ..config.plan import PartSpec
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    def __init__(self, mixer, feed_forward, norm: PartSpec, mixer_norm_name: str, feed_forward_norm_name: str):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm = build_part("norm", norm)
        self.feed_forward_norm = build_part("norm", norm)
        self.mixer_norm_name, self.feed_forward_norm_name = mixer_norm_name, feed_forward_norm_name

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        specs.update(self.mixer_norm.weight_specs(prefix + self.mixer_norm_name))
        specs.update(self.feed_forward_norm.weight_specs(prefix + self.feed_forward_norm_name))
        specs.update(self.mixer.weight_specs(prefix))
        specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.mixer_norm.bind(weights, prefix + self.mixer_norm_name, dtype, device)
        self.feed_forward_norm.bind(weights, prefix + self.feed_forward_norm_name, dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        self.feed_forward.bind(weights, prefix, dtype, device)

    def forward(self, residual, delta, ctx, cache):
        normed = ctx.scratch.get("block.normed", residual.shape, ctx.dtype)
        self.mixer_norm(residual, normed, delta)
        mixed = self.mixer.forward(normed, ctx, cache)
        self.feed_forward_norm(residual, normed, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


class NormedBranch:
    """A sublayer's output (compute type) that is still to be normalised with `norm` and added to the float32 stream."""

    def __init__(self, branch, norm):
        self.branch, self.norm = branch, norm


def settle(residual, pending, norm=None, out=None):
    """stream += norm_b(branch) for a pending `NormedBranch` (None: nothing to add), and, with `norm` and `out`,
    out = norm(stream) of the sum: one kernel."""
    from ..csrc import ops
    if pending is not None and not isinstance(pending, NormedBranch):
        raise TypeError("a float32 stream takes a NormedBranch as its pending sum")
    if pending is None and norm is None:
        return out
    return ops.sandwich_norm(residual, pending.branch if pending else None, pending.norm.weight if pending else None,
                             pending.norm.eps if pending else 0.0, norm.weight if norm else None,
                             norm.eps if norm else 0.0, out)


class SandwichNormBlock(Part):
    stream_dtype = "float32"

    def __init__(self, mixer, feed_forward, norm: PartSpec, names=("norm1", "norm1b", "norm2", "norm2b")):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.names = tuple(names)
        self.norms = [build_part("norm", norm) for _ in range(4 if feed_forward is not None else 2)]

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        for part, name in zip(self.norms, self.names):
            specs.update(part.weight_specs(prefix + name))
        specs.update(self.mixer.weight_specs(prefix))
        if self.feed_forward is not None:
            specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        for part, name in zip(self.norms, self.names):
            part.bind(weights, prefix + name, dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        if self.feed_forward is not None:
            self.feed_forward.bind(weights, prefix, dtype, device)

    def forward(self, residual, delta, ctx, cache):
        normed = ctx.scratch.get("block.normed", residual.shape, ctx.dtype)
        settle(residual, delta, self.norms[0], normed)
        pending = NormedBranch(self.mixer.forward(normed, ctx, cache), self.norms[1])
        if self.feed_forward is None:
            return residual, pending
        settle(residual, pending, self.norms[2], normed)
        return residual, NormedBranch(self.feed_forward.forward(normed, ctx), self.norms[3])


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
