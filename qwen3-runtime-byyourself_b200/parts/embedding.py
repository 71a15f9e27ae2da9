"""Token embedding and output head as parts.

Embedding: a row gather (src/ops/embedding.cu:38-52).  Head: logits = x . W^T with W
either `lm_head.weight` or, for tied checkpoints, the embedding table, in which case
`lm_head.weight` is not read (src/model/weights.cpp:116-118,198-204).  The reference
rounds logits to bfloat16 (src/ops/linear.cpp:118); here they leave the product as
float32.

Parameters beyond Qwen3: the embedding can be multiplied by a constant (`scale`; its output is
then float32, the hidden state of a model that keeps it in 32-bit); the logits can be
multiplied by a constant (`scale`) and capped smoothly (`softcap`: z <- c tanh(z / c)); the
tensors' names are the prefix plus `tensor`.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, scale: Optional[float] = None, tensor: str = "weight",
                 copies: int = 1):
        """`copies` > 1: every token's row is written that many times side by side (out [N, copies * hidden])."""
        self.vocab_size, self.hidden_size, self.copies = int(vocab_size), int(hidden_size), int(copies)
        self.scale = None if scale is None else float(scale)
        self.tensor = tensor
        self.table = None

    def weight_specs(self, prefix: str) -> dict:
        return {prefix + self.tensor: WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.table = weights[prefix + self.tensor].contiguous()

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        if self.copies > 1:
            return ops.embedding_streams(token_ids, self.table, out, 1.0 if self.scale is None else self.scale, self.copies)
        if out.dtype == torch.float32 and (self.scale is not None or self.table.dtype != torch.float32):
            return ops.embedding_scaled(token_ids, self.table, out, 1.0 if self.scale is None else self.scale)
        if self.scale is not None:
            raise ops.KernelError("a scaled embedding writes a float32 hidden state")
        return ops.embedding(token_ids, self.table, out)


class LMHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None, scale: Optional[float] = None,
                 softcap: Optional[float] = None, tensor: str = "weight"):
        self.vocab_size, self.hidden_size, self.tied_to = int(vocab_size), int(hidden_size), tied_to
        self.scale = 1.0 if scale is None else float(scale)
        self.softcap = float(softcap) if softcap else 0.0
        self.tensor = tensor
        self.weight = None

    def weight_specs(self, prefix: str) -> dict:
        return {} if self.tied_to else {prefix + self.tensor: WeightSpec((self.vocab_size, self.hidden_size))}

    def ignorable(self, prefix: str):
        return [prefix + self.tensor] if self.tied_to else []

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.weight = weights[self.tied_to if self.tied_to else prefix + self.tensor].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        linear(x, self.weight, out)
        if self.scale != 1.0 or self.softcap:
            ops.scale_softcap(out, self.scale, self.softcap)
        return out


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
