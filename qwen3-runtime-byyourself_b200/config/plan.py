"""Architecture-independent description of a model: which parts, in which order.

A configuration class (one per architecture) turns its config.json into a
`ModelPlan`.  Everything below the plan - parts, cache, step function, replay,
generation - reads the plan only and never the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part by the name it was registered under, with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement that holds a mixer and a feed-forward.

    `prefix` is the checkpoint-name prefix of the layer's tensors.  `cache_from`
    names another layer whose cache this layer's mixer reads instead of owning
    one (None: the layer owns its cache).
    """
    block: PartSpec
    mixer: PartSpec
    feed_forward: Optional[PartSpec]      # None: the layer has no feed-forward (its block must allow that)
    prefix: str
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class StreamStep:
    """A part that rewrites the hidden state between layers from the state and the embedding's output
    (family `stream`): it runs right before entry `before_run` of the plan's `order`.  `name` is the
    checkpoint name of its tensor (or the prefix of its tensors)."""
    before_run: int
    part: PartSpec
    name: str


@dataclass(frozen=True)
class ModelPlan:
    """The whole model as data.

    `order` is the sequence in which layers run; it may name a layer twice.  `caches` gives, for
    every entry of `order`, the number of the cache (pages and state) that run uses: a layer that
    runs several times with the same weights can keep one cache per run.  Numbers below the number
    of layers are the layers' own caches, numbers from there on are further ones of the same kind
    as the layer's that uses them.  None: every run of a layer uses the layer's own cache.
    `stream_steps` run between layers; `residual_dtype` "float32" keeps the hidden state between
    the parts in 32-bit whatever the compute type (None: in the compute type).  With `streams` > 1 the
    hidden state is that many rows per token (the embedding fills them alike, the blocks mix them, and
    the last block's `finish` sums them).
    """
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    embedding_prefix: str
    layers: List[LayerSpec]
    order: List[int]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    stop_token_ids: List[int] = field(default_factory=list)
    caches: Optional[List[int]] = None
    stream_steps: List[StreamStep] = field(default_factory=list)
    residual_dtype: Optional[str] = None
    final_norm_name: Optional[str] = None     # the final norm's tensor (None: final_norm_prefix + "weight")
    streams: int = 1                          # copies of the hidden state that travel side by side ([tokens, streams, hidden])

    def cache_of_run(self, run: int) -> int:
        return self.order[run] if self.caches is None else self.caches[run]

    def cache_owners(self) -> List[Optional[int]]:
        """For every cache number, the layer whose mixer states what the cache holds (None: unused)."""
        owners: List[Optional[int]] = list(range(len(self.layers)))
        for run, layer in enumerate(self.order):
            unit = self.cache_of_run(run)
            owners.extend([None] * (unit + 1 - len(owners)))
            owners[unit] = layer
        return owners

    def __post_init__(self):
        n = len(self.layers)
        if self.caches is not None:
            if len(self.caches) != len(self.order):
                raise ValueError("caches names one cache for every entry of order")
            for run, unit in enumerate(self.caches):
                if unit < 0 or (unit < n and unit != self.order[run]):
                    raise ValueError(f"run {run}: cache {unit} is another layer's own")
        for step in self.stream_steps:
            if not 0 <= step.before_run < len(self.order):
                raise ValueError(f"a stream step before run {step.before_run}, but the plan has {len(self.order)} runs")
        if self.streams < 1 or (self.streams > 1 and self.residual_dtype != "float32"):
            raise ValueError("streams is at least 1; several streams are kept in float32")
        if self.residual_dtype not in (None, "float32"):
            raise ValueError("residual_dtype is None (the compute type) or 'float32'")
        for i in self.order:
            if not 0 <= i < n:
                raise ValueError(f"order names layer {i}, but the plan has {n} layers")
        for i, layer in enumerate(self.layers):
            src = layer.cache_from
            if src is None:
                continue
            if not 0 <= src < n or src == i or self.layers[src].cache_from is not None:
                raise ValueError(f"layer {i}: cache_from={src} must name another layer that owns its cache")
            if src not in self.order or i not in self.order or self.order.index(src) > self.order.index(i):
                raise ValueError(f"layer {i} reads the cache of layer {src}, which has to run first")
