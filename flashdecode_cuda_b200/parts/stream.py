"""Operations on the whole residual stream between layers."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Part, Runtime
from .linear import matmul


class StreamOp(Part):
    """``forward(ctx, resid, delta, embedded, index=None) -> delta``: ``resid`` [T, H] float32 is the residual
    stream, ``delta`` the output of the last sub-layer that has not been added to it yet (or None), ``embedded`` the
    embedding output of the step, ``index`` the number the schedule entry gives (``RunSpec.before_index``: which
    pass of a loop this is).  The operation leaves the new stream in ``resid`` and returns what is still to be
    added to it (None: nothing).  ``needs_embedded`` False: the model need not keep the embedding output."""
    kind = "stream_op"
    accepts_parts = False
    needs_embedded = True


@register_part("stream_op", "reinject_embedding")
class ReinjectEmbedding(StreamOp):
    """x <- W [x ; x0]: the stream and the embedding output side by side through one matrix ``<tensor>``
    [H, 2H] (x's columns first).  The sum that completes x and the result are float32; the product runs in the
    model's dtype."""

    def __init__(self, prefix: str, hidden_size: int, tensor: Optional[str] = None):
        self.name = tensor or f"{prefix}.weight"
        self.hidden_size = hidden_size

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.hidden_size, 2 * self.hidden_size), init="unit")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = tensors[self.name]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.weight

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor], embedded: torch.Tensor,
                index: Optional[int] = None):
        both = ctx.ws.get("reinject_in", (ctx.T, 2 * self.hidden_size), self.rt.dtype)
        K.add_concat(delta, resid, embedded, both)
        matmul(both, self.weight, None, resid, status=self.rt.status)
        return None


@register_part("stream_op", "add_pass_vector")
class AddPassVector(StreamOp):
    """x <- x + v[index]: a vector per pass of a loop, rows of ``<tensor>`` [passes, H], added to every token's
    stream right before the pass's first layer.  The pending output of the layer before is added here too, times
    ``delta_scale`` (a model whose sub-layers enter the stream times a constant).  All float32."""

    needs_embedded = False

    def __init__(self, prefix: str, hidden_size: int, passes: int, tensor: Optional[str] = None,
                 delta_scale: Optional[float] = None):
        self.name = tensor or f"{prefix}.weight"
        self.hidden_size, self.passes = hidden_size, passes
        self.delta_scale = 1.0 if delta_scale is None else float(delta_scale)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.passes, self.hidden_size), "vector", init="bias")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.vectors = tensors[self.name].float().contiguous()

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor], embedded: Optional[torch.Tensor],
                index: Optional[int] = None):
        if index is None or not (0 <= index < self.passes):
            raise ValueError(f"{self.name}: pass {index} of {self.passes}")
        if delta is not None and delta.dim() == 3:
            raise ValueError(f"{self.name}: partial sums were handed to a part that did not ask for them")
        K.add_row_vector(delta, resid, self.vectors[index], self.delta_scale)
        return None
