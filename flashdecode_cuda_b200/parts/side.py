"""What a layer adds to the residual stream from the token itself: a narrow second embedding, gated by the stream."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Part, Runtime
from .linear import matmul

# Up to this many tokens the whole contribution is two launches whose CTAs each read their share of the small matrices
# once per token; above it the two products go through the matrix-product kernels.
SIDE_FUSED_MAX_TOKENS = 64


@register_part("table", "token_rows")
class TokenRows(Part):
    """A lookup table [vocab, columns] that several parts read by token id, each its own columns.  Declared once,
    handed to the parts that name it (``table="name"`` against ``ModelBlueprint.tables``)."""
    kind = "table"

    def __init__(self, prefix: str, vocab_size: int, columns: int, tensor: Optional[str] = None):
        self.name = tensor or f"{prefix}.weight"
        self.vocab_size, self.columns = vocab_size, columns
        self.table = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.columns), "matrix", init="unit_rows")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.table = tensors[self.name]


class SideInput(Part):
    """``forward(ctx, resid, delta) -> delta``: runs at the end of a layer.  It adds the layer's pending output
    ``delta`` to the stream ``resid`` [T, H] (float32) itself, because it reads the stream as it stands after the
    layer's sub-layers, and returns its own contribution, still to be added by whoever norms next."""
    kind = "side_input"


@register_part("side_input", "gated_token_rows")
class GatedTokenRows(SideInput):
    """For the stream x [T, H] after a layer's sub-layers and the layer's columns e of a token table:

        g = gelu_tanh(W_gate x) * e[token]          W_gate [dim, H]
        y = W_proj g                                W_proj [H, dim]
        out = y / sqrt(mean(y^2) + eps) * w         (w [H], a plain RMS-norm weight)

    x itself is completed here: x = resid + delta_scale * delta, written back in float32.  The products run in the
    model's dtype with float32 sums; the activation, the norm and ``out`` are float32.  Tensors ``<prefix>.gate``,
    ``.proj``, ``.norm``; the table belongs to a ``table`` part, of which this part reads ``dim`` columns from
    ``first_col`` on."""

    def __init__(self, prefix: str, hidden_size: int, dim: int, table, first_col: int, eps: float,
                 delta_scale: Optional[float] = None):
        if dim < 1 or first_col < 0 or first_col + dim > table.columns:
            raise ValueError(f"{prefix}: columns {first_col} .. {first_col + dim} of a table of {table.columns}")
        self.prefix, self.hidden_size, self.dim, self.table, self.first_col = prefix, hidden_size, dim, table, first_col
        self.eps = float(eps)
        self.delta_scale = 1.0 if delta_scale is None else float(delta_scale)

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        return [TensorSpec(f"{p}.gate", (self.dim, H), init="unit"), TensorSpec(f"{p}.proj", (H, self.dim), init="unit"),
                TensorSpec(f"{p}.norm", (H,), "vector", init="norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        self.w_gate, self.w_proj = tensors[f"{p}.gate"], tensors[f"{p}.proj"]
        self.norm_w = tensors[f"{p}.norm"].float().contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate.numel() + self.w_proj.numel()) * self.w_gate.element_size() + self.norm_w.numel() * 4

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        T, H, ws, rt = ctx.T, self.hidden_size, ctx.ws, self.rt
        if delta is not None and delta.dim() == 3:
            raise ValueError(f"{self.prefix}: partial sums were handed to a part that did not ask for them")
        out = ws.get("side_out", (T, H), torch.float32)
        table = self.table.table
        # float32 keeps the matrix products' fixed summation order whatever the step holds
        if (rt.dtype == torch.bfloat16 and T <= SIDE_FUSED_MAX_TOKENS
                and H + self.dim + 8 <= K.TOKEN_SIDE_ROW_MAX_FLOATS):
            K.token_side_row(delta, resid, self.delta_scale, ctx.tokens, table, self.first_col, self.w_gate, self.w_proj,
                             self.norm_w, self.eps, out, rt.status, scratch=ws.get("side_z", (T, self.dim), torch.float32))
            return out
        x = ws.get("side_x", (T, H), rt.dtype)
        K.add_cast(delta, resid, x, self.delta_scale)
        z = ws.get("side_z", (T, self.dim), torch.float32)
        matmul(x, self.w_gate, None, z, status=rt.status)
        g = ws.get("side_g", (T, self.dim), rt.dtype)
        K.side_gate_mul(z, ctx.tokens, table, self.first_col, g, rt.status)
        y = ws.get("side_y", (T, H), torch.float32)
        matmul(g, self.w_proj, None, y, status=rt.status)
        K.add_rmsnorm(None, y, self.norm_w, self.eps, out, write_resid=False)
        return out
