"""Token embedding: the start of the residual stream."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Embedding, Runtime


@register_part("embedding", "token_table")
class TokenEmbedding(Embedding):
    """resid[t] = table[token[t]], unscaled (engine/model.py:166,255 of
    davidjoyme/flashdecode-cuda), written as float32; into every lane of a
    residual stream that has several ([T, lanes * hidden_size]).  ``scale``:
    the row is multiplied by it (in float32) as it enters the stream; the table
    itself, which a tied head reads, stays as stored."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tensor: Optional[str] = None,
                 scale: Optional[float] = None):
        self.name = tensor or f"{prefix}.weight"        # ``tensor``: the table's full name where it is not <prefix>.weight
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.scale = 1.0 if scale is None else float(scale)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "matrix", init="embedding")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.table = tensors[self.name]

    def forward(self, ctx, resid: torch.Tensor) -> None:
        K.embed(ctx.tokens, self.table, resid, self.rt.status, self.scale)
