"""Typed configuration of the Lagulorn decoder, read from its config.json.

A Lagulorn model is a list of layers; each has one of two mixers and, optionally, a feed-forward that is
dense or a mixture of experts.  A layer may borrow another layer's weights and still keep a cache or state
of its own.  The hidden state may travel as several streams that every sublayer reads as a weighted sum and
writes back through a small mixing matrix (hyper-connections).  What the file gives, key by key:

  architecture        "Lagulorn"
  vocab, width        sizes of the embedding table and of the hidden state
  embedding.scale     the embedding's output is multiplied by it
  norm.eps            eps of every RMS norm (inside the root); norm weights are stored around zero (1 + w)
  residual_mult       every sublayer's output is multiplied by it before it is added
  streams             number of copies of the hidden state (absent: one, with a plain residual sum)
  layers[i].type      "attention": mixer {heads, kv_heads, dim, vdim, scale, diff, mask {size}}: differential
                      attention (two softmax maps per head over the same values, o = a1 - lambda a2), per-head
                      norms of q and k, a sliding window, no rotation
                      "lightning": mixer {heads, dim, vdim, decay [heads]}: linear attention with a per-head
                      decay and a float32 state per sequence
  layers[i].mlp       {kind "dense", ff} | {kind "moe", expert {ff, limit}, router {experts, top, identity,
                      groups {count, keep}}} | null
  layers[i].weights_of   j: the layer has no tensors of its own and runs with layer j's

Optional keys (`embedding`, `residual_mult`, `streams`, `mask`, `mlp`, `router.identity`, `router.groups`,
`weights_of`) may be null or absent: the mechanism is then not there.  `plan()` states the model as data
for the parts, the cache and the step function.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .dozazen import MAX_POSITIONS, _get, _opt
from .plan import LayerSpec, ModelPlan, PartSpec
from .registry import ConfigError, register_architecture

MAX_STREAMS = 16


@dataclass(frozen=True)
class LagulornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    streams: Optional[int]
    layers: List[Dict[str, Any]]            # as in the file, checked
    torch_dtype: str = "bfloat16"

    architecture = "Lagulorn"

    @classmethod
    def from_dict(cls, root: dict) -> "LagulornConfig":
        if not isinstance(root, dict):
            raise ConfigError("model config root must be a JSON object")
        name = root.get("architecture", (root.get("architectures") or [None])[0])
        if name != cls.architecture:
            raise ConfigError(f"only {cls.architecture} is read by this class, not {name!r}")
        layers = root.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty array")
        embedding = _opt(root, "embedding", dict) or {}
        scale, mult = _opt(embedding, "scale", float, "embedding."), _opt(root, "residual_mult", float)
        config = cls(
            vocab=_get(root, "vocab", int),
            width=_get(root, "width", int),
            embedding_scale=1.0 if scale is None else scale,
            norm_eps=_get(_get(root, "norm", dict), "eps", float, "norm."),
            residual_mult=1.0 if mult is None else mult,
            streams=_opt(root, "streams", int),
            layers=copy.deepcopy(layers),
            torch_dtype=_opt(root, "torch_dtype", str) or "bfloat16",
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError("torch_dtype is bfloat16 or float32")
        if self.streams is not None and not 1 <= self.streams <= MAX_STREAMS:
            raise ConfigError(f"streams must be between 1 and {MAX_STREAMS}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"{where[:-1]} must be an object")
            kind = _get(layer, "type", str, where)
            m, w = _get(layer, "mixer", dict, where), where + "mixer."
            heads, dim, vdim = _get(m, "heads", int, w), _get(m, "dim", int, w), _get(m, "vdim", int, w)
            if heads <= 0 or not 0 < dim <= 256 or not 0 < vdim <= 256:
                raise ConfigError(f"{w}heads {heads}, dim {dim}, vdim {vdim}: positive, head sizes up to 256")
            if kind == "attention":
                kv = _get(m, "kv_heads", int, w)
                if kv <= 0 or heads % kv:
                    raise ConfigError(f"{w}heads must be a positive multiple of kv_heads")
                _get(m, "scale", float, w)
                _get(m, "diff", float, w)
                mask = _opt(m, "mask", dict, w)
                if mask is not None and _get(mask, "size", int, w + "mask.") <= 0:
                    raise ConfigError(f"{w}mask.size must be positive")
            elif kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != heads:
                    raise ConfigError(f"{w}decay must list one number per head")
                for j, value in enumerate(decay):
                    if isinstance(value, bool) or not isinstance(value, (int, float)) or not 0.0 <= float(value) <= 1.0:
                        raise ConfigError(f"{w}decay[{j}] must be a number from 0 to 1")
            else:
                raise ConfigError(f"{where}type: 'attention' or 'lightning', not {kind!r}")
            mlp = _opt(layer, "mlp", dict, where)
            if mlp is not None:
                self._check_mlp(mlp, where + "mlp.")
            owner = _opt(layer, "weights_of", int, where)
            if owner is not None:
                if not 0 <= owner < len(self.layers) or owner == i or self.layers[owner].get("weights_of") is not None:
                    raise ConfigError(f"{where}weights_of must name another layer that has tensors of its own")
                if layer["type"] != self.layers[owner].get("type"):
                    raise ConfigError(f"{where}weights_of: layer {owner} is of another type")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = _get(mlp, "kind", str, where)
        if kind == "dense":
            if _get(mlp, "ff", int, where) <= 0:
                raise ConfigError(f"{where}ff must be positive")
            return
        if kind != "moe":
            raise ConfigError(f"{where}kind: 'dense' or 'moe', not {kind!r}")
        expert = _get(mlp, "expert", dict, where)
        if _get(expert, "ff", int, where + "expert.") <= 0 or not _get(expert, "limit", float, where + "expert.") > 0:
            raise ConfigError(f"{where}expert needs a positive ff and a positive limit")
        r, w = _get(mlp, "router", dict, where), where + "router."
        experts, top, identity = _get(r, "experts", int, w), _get(r, "top", int, w), _opt(r, "identity", int, w) or 0
        if experts < 0 or identity < 0 or experts + identity <= 0 or not 0 < top <= experts + identity:
            raise ConfigError(f"{w}needs experts + identity > 0 and 0 < top <= experts + identity")
        groups = _opt(r, "groups", dict, w)
        if groups is not None:
            count, keep = _get(groups, "count", int, w + "groups."), _get(groups, "keep", int, w + "groups.")
            if count <= 0 or (experts + identity) % count or not 0 < keep <= count:
                raise ConfigError(f"{w}groups: count must divide experts + identity, 0 < keep <= count")
            if keep * ((experts + identity) // count) < top:
                raise ConfigError(f"{w}groups: the kept groups hold fewer than top experts")

    def to_dict(self) -> dict:
        """The keys of a config.json that `from_dict` reads back to an equal object."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": copy.deepcopy(self.layers), "torch_dtype": self.torch_dtype}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    # -- the model as data
    def plan(self) -> ModelPlan:
        H = self.width
        norm = PartSpec("rms_norm", {"size": H, "eps": self.norm_eps, "one_plus": True})
        owners = [i for i, layer in enumerate(self.layers) if layer.get("weights_of") is None]
        layers = []
        for i in owners:
            layer = self.layers[i]
            m = layer["mixer"]
            if layer["type"] == "attention":
                mixer = PartSpec("differential_attention", {
                    "hidden_size": H, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                    "value_dim": m["vdim"], "scale": float(m["scale"]), "diff": float(m["diff"]),
                    "window": m["mask"]["size"] if m.get("mask") else None, "eps": self.norm_eps, "prefix": "mix.",
                    "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})
            else:
                mixer = PartSpec("lightning_attention", {
                    "hidden_size": H, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                    "decay": [float(v) for v in m["decay"]], "eps": self.norm_eps, "prefix": "mix."})
            feed_forward, mlp = None, layer.get("mlp")
            if mlp is not None and mlp["kind"] == "dense":
                feed_forward = PartSpec("dense_mlp", {"hidden_size": H, "intermediate_size": mlp["ff"], "prefix": "mlp.",
                                                      "activation": "gelu", "names": {"up": "up", "down": "down"}})
            elif mlp is not None:
                r = mlp["router"]
                groups = r.get("groups") or {}
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": H, "intermediate_size": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]),
                    "experts": r["experts"], "identity": r.get("identity") or 0, "top": r["top"],
                    "group_count": groups.get("count", 1), "group_keep": groups.get("keep", 1), "prefix": "mlp."})
            block = PartSpec("hyper_connections", {"norm": norm, "streams": self.streams, "residual_mult": self.residual_mult,
                                                   "hidden_size": H})
            layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=feed_forward, prefix=f"l{i}."))
        n, order, caches = len(layers), [], []
        extra = n
        for i, layer in enumerate(self.layers):
            owner = layer.get("weights_of")
            if owner is None:
                order.append(owners.index(i))
                caches.append(owners.index(i))
            else:                                            # borrowed weights, a cache or state of its own
                order.append(owners.index(owner))
                caches.append(extra)
                extra += 1
        copies = self.streams or 1
        return ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=H, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": H, "scale": self.embedding_scale,
                                                   "tensor": "", "copies": copies}),
            embedding_prefix="embed", layers=layers, order=order, caches=caches, streams=copies,
            residual_dtype="float32", final_norm=norm, final_norm_prefix="final.", final_norm_name="final.norm",
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": H, "tensor": ""}),
            head_prefix="head", stop_token_ids=[],
        )


register_architecture(LagulornConfig.architecture, LagulornConfig)
