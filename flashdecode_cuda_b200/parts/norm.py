"""Norms fused with the deferred residual add: RMSNorm and Dynamic Tanh."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Norm, Runtime


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """resid += delta; out = resid * rsqrt(mean(resid^2) + eps) * weight.

    The formula of ``rmsnorm_residual`` in davidjoyme/flashdecode-cuda
    (engine/ops.py:61-79, kernels/rmsnorm.cu:70-132).  There the sum is rounded
    to bfloat16 before it is squared and kept; here the residual stream stays in
    float32 and everything up to the final store is float32.
    """

    accepts_parts = True        # the kernel adds up to four float partial sums in order while it adds the residual

    def __init__(self, prefix: str, size: int, eps: float, unit_offset: bool = False, tensor: Optional[str] = None,
                 optional: bool = False, delta_scale: Optional[float] = None):
        """``unit_offset``: the checkpoint holds the gain's offset from one and the norm multiplies by 1 + weight (added in
        float32 when the weights are bound).  ``tensor``: the weight's full name where it is not
        ``<prefix>.weight``.  ``optional``: a checkpoint may lack the weight (a norm that never runs).
        ``delta_scale``: a model whose sub-layers enter the stream times a constant, x += c f(norm(x)): the pending
        output is multiplied by c (in float32) as this norm adds it."""
        self.name = tensor or f"{prefix}.weight"
        self.size, self.eps, self.unit_offset, self.optional = size, float(eps), bool(unit_offset), bool(optional)
        self.delta_scale = 1.0 if delta_scale is None else float(delta_scale)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), "vector", optional=self.optional,
                           init="norm_zero" if self.unit_offset else "norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = tensors.get(self.name) if self.optional else tensors[self.name]
        if self.unit_offset and self.weight is not None:
            self.weight = (1.0 + self.weight.float()).contiguous()

    def forward(self, ctx, delta: Optional[torch.Tensor], resid: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                write_resid: bool = True, n_parts: int = 1) -> None:
        K.add_rmsnorm(delta, resid, self.weight, self.eps, out, rows=rows, n_out=n_out,
                      write_resid=write_resid, n_parts=n_parts, delta_scale=self.delta_scale)


@register_part("norm", "dyn_tanh")
class DynTanh(Norm):
    """resid += delta; out = tanh(alpha * resid) * weight + bias, with a learned scalar alpha: a norm that computes no
    mean and no variance.  Tensors ``<tensor>`` (weight), ``<tensor>.b`` and ``<tensor>.alpha`` (a scalar).  The sum,
    the tanh and the affine map are float32 in both dtypes; weight and bias are kept in float32."""

    def __init__(self, prefix: str, size: int, tensor: Optional[str] = None, optional: bool = False):
        self.name = tensor or f"{prefix}.weight"
        self.size, self.optional = size, bool(optional)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), "vector", optional=self.optional, init="norm"),
                TensorSpec(f"{self.name}.b", (self.size,), "vector", optional=self.optional, init="bias"),
                TensorSpec(f"{self.name}.alpha", (), "vector", optional=self.optional, init="half")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = self.bias = None
        self.alpha = 1.0
        if self.name in tensors:
            self.weight = tensors[self.name].float().contiguous()
            self.bias = tensors[f"{self.name}.b"].float().contiguous()
            self.alpha = float(tensors[f"{self.name}.alpha"].float().item())     # a kernel argument from now on

    def forward(self, ctx, delta: Optional[torch.Tensor], resid: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                write_resid: bool = True, n_parts: int = 1) -> None:
        K.add_dyn_tanh(delta, resid, self.weight, self.bias, self.alpha, out, rows=rows, n_out=n_out,
                       write_resid=write_resid)
