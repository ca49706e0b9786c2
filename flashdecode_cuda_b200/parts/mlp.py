"""Dense feed-forwards: gated (SwiGLU and its relatives) and plain with a parametric activation."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime
from .linear import GEMV_MAX_ROWS, MAX_PARTS, fused_prompt_gemm, matmul, stream_gemm


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """down( silu(gate(x)) * up(x) ), no biases (engine/model.py:213-216 and
    engine/ops.py:201-204 of davidjoyme/flashdecode-cuda).  gate and up are one
    [2I, H] matrix here, so they are one product."""

    offers_parts = True     # forward(..., parts_ok=True) may return float partial sums [parts, T, H]

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size, self.inter = prefix, hidden_size, intermediate_size

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I = self.prefix, self.hidden_size, self.inter
        return [TensorSpec(f"{p}.gate_proj.weight", (I, H)),
                TensorSpec(f"{p}.up_proj.weight", (I, H)),
                TensorSpec(f"{p}.down_proj.weight", (H, I))]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p, I = self.prefix, self.inter
        gate, up = tensors.pop(f"{p}.gate_proj.weight"), tensors.pop(f"{p}.up_proj.weight")
        # tiles of 16 rows: 8 gate rows, then the 8 up rows of the same outputs, so the decode
        # kernel's thread that holds gate_i also holds up_i (csrc/gemv_mma.cu)
        self.tiled = I % 8 == 0
        if self.tiled:
            H = gate.shape[1]
            self.w_gate_up = torch.stack([gate.view(I // 8, 8, H), up.view(I // 8, 8, H)], dim=1) \
                .reshape(2 * I, H).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[f"{p}.down_proj.weight"]

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_gate_up

    def forward(self, ctx, x: torch.Tensor, parts_ok: bool = False) -> torch.Tensor:
        """delta [T, H]; with ``parts_ok`` (the caller's consumer adds partial sums up) a decode step's down
        projection may come back as float32 [parts, T, H] instead."""
        T, ws = ctx.T, ctx.ws
        act = ws.get("ffn_act", (T, self.inter), x.dtype)
        if (self.tiled and x.dtype == torch.bfloat16 and T <= GEMV_MAX_ROWS
                and K.gemv_splits(T, 2 * self.inter, self.hidden_size, 1, allow_split=False) == 1):
            K.gemv(x, self.w_gate_up, None, act, K.GEMV_GATED)          # product and silu(gate) * up in one kernel
        elif self.tiled and x.dtype == torch.bfloat16 and stream_gemm(T, 2 * self.inter, self.hidden_size):
            K.gemm_stream(x, self.w_gate_up, None, act, gated=True, status=self.rt.status)      # 17 to 128 rows: the same fusion
        elif self.tiled and x.dtype == torch.bfloat16 and fused_prompt_gemm(T, 2 * self.inter, self.hidden_size):
            K.gemm_tc(x, self.w_gate_up, None, act, gated=True, status=self.rt.status)     # prompts: tcgen05, same fusion
        else:
            gu = ws.get("gate_up", (T, 2 * self.inter), x.dtype)
            matmul(x, self.w_gate_up, None, gu, status=self.rt.status)
            K.silu_mul(gu, act, tiled=self.tiled)
        out = ws.get("ffn_out", (T, self.hidden_size), x.dtype)
        parts = None
        if parts_ok and T <= GEMV_MAX_ROWS:
            parts = ws.get("ffn_out_parts", (MAX_PARTS, T, self.hidden_size), torch.float32)
        return matmul(act, self.w_down, None, out, target_ctas=4 * self.rt.sm_count, parts=parts, status=self.rt.status,
                      upcoming=ctx.upcoming)


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    """down( act(gate(x)) * up(x) ) with a choice of activation and biases on all three projections.

    ``activation``: ``"silu"`` or ``"gelu_tanh"`` (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))).  ``bias``: every
    projection has one.  Tensors ``<prefix>.gate`` / ``.up`` / ``.down`` (stored [out, in]) and, with biases,
    ``.gate.b`` / ``.up.b`` / ``.down.b``.  gate and up are one packed product; the activation is computed in float32
    from the product's float sums (bfloat16: in the product's epilogue, rows of the packed matrix in tiles of 8 gate +
    8 up) or from its output (float32) and rounded once.
    """

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh",
                 bias: bool = True):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"{prefix}: unknown activation {activation!r}; known: silu, gelu_tanh")
        self.prefix, self.hidden_size, self.inter = prefix, hidden_size, intermediate_size
        self.activation, self.bias = activation, bool(bias)
        self.kind = K.GLU_KINDS[activation]

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I = self.prefix, self.hidden_size, self.inter
        specs = [TensorSpec(f"{p}.gate", (I, H), init="unit"), TensorSpec(f"{p}.up", (I, H), init="unit"),
                 TensorSpec(f"{p}.down", (H, I), init="unit")]
        if self.bias:
            specs += [TensorSpec(f"{p}.gate.b", (I,), "vector", init="bias"),
                      TensorSpec(f"{p}.up.b", (I,), "vector", init="bias"),
                      TensorSpec(f"{p}.down.b", (H,), "vector", init="bias")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        I = self.inter
        # bfloat16: tiles of 16 rows, 8 gate rows and the 8 up rows of the same outputs, so that the thread of a product's
        # epilogue that holds gate_i also holds up_i
        self.tiled = rt.dtype == torch.bfloat16 and I % 8 == 0

        def pack(g, u):
            if not self.tiled:
                return torch.cat([g, u], dim=0).contiguous()
            return torch.stack([g.reshape(I // 8, 8, -1), u.reshape(I // 8, 8, -1)], dim=1).reshape(2 * I, *g.shape[1:]).contiguous()
        self.w_gate_up = pack(tensors.pop(f"{p}.gate"), tensors.pop(f"{p}.up"))
        self.w_down = tensors[f"{p}.down"]
        self.b_gate_up = self.b_down = None
        if self.bias:
            self.b_gate_up = pack(tensors.pop(f"{p}.gate.b"), tensors.pop(f"{p}.up.b"))
            self.b_down = tensors[f"{p}.down.b"]

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_gate_up

    def forward(self, ctx, x: torch.Tensor, parts_ok: bool = False) -> torch.Tensor:
        T, ws = ctx.T, ctx.ws
        act = ws.get("ffn_act", (T, self.inter), x.dtype)
        N2, H = 2 * self.inter, self.hidden_size
        if self.tiled and T <= GEMV_MAX_ROWS and K.gemv_splits(T, N2, H, 1, allow_split=False) == 1:
            K.gemv(x, self.w_gate_up, self.b_gate_up, act, K.GEMV_GATED_GELU if self.kind else K.GEMV_GATED)
        elif self.tiled and stream_gemm(T, N2, H):
            K.gemm_stream(x, self.w_gate_up, self.b_gate_up, act, gated=self.activation, status=self.rt.status)
        elif self.tiled and fused_prompt_gemm(T, N2, H):
            K.gemm_tc(x, self.w_gate_up, self.b_gate_up, act, gated=self.activation, status=self.rt.status)
        else:
            gu = ws.get("gate_up", (T, N2), x.dtype)
            matmul(x, self.w_gate_up, self.b_gate_up, gu, status=self.rt.status)
            K.glu_mul(gu, act, self.kind, tiled=self.tiled)
        out = ws.get("ffn_out", (T, self.hidden_size), x.dtype)
        return matmul(act, self.w_down, self.b_down, out, target_ctas=4 * self.rt.sm_count, status=self.rt.status,
                      upcoming=ctx.upcoming)


@register_part("feed_forward", "dense_act")
class DenseActMLP(FeedForward):
    """down( act(up(x)) ), no gate and no biases, with the two-parameter activation ``quad_exp``:

        act(z) = softplus(p) z^2 + z / 2                          for z > 0
                 (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2     for z <= 0

    (p, q) are the tensor ``<prefix>.act`` [2].  Tensors ``<prefix>.up`` / ``.down`` (stored [out, in]).  The
    activation is computed in float32 and rounded once."""

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "quad_exp"):
        if activation != "quad_exp":
            raise ValueError(f"{prefix}: unknown activation {activation!r}; known: quad_exp")
        self.prefix, self.hidden_size, self.inter, self.activation = prefix, hidden_size, intermediate_size, activation

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I = self.prefix, self.hidden_size, self.inter
        return [TensorSpec(f"{p}.up", (I, H), init="unit"), TensorSpec(f"{p}.down", (H, I), init="unit"),
                TensorSpec(f"{p}.act", (2,), "vector", init="half")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        self.w_up, self.w_down = tensors[f"{p}.up"], tensors[f"{p}.down"]
        self.pq = tensors.pop(f"{p}.act").float().contiguous()

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_up

    def forward(self, ctx, x: torch.Tensor, parts_ok: bool = False) -> torch.Tensor:
        T, ws = ctx.T, ctx.ws
        up = ws.get("ffn_up", (T, self.inter), x.dtype)
        matmul(x, self.w_up, None, up, status=self.rt.status)
        act = ws.get("ffn_act", (T, self.inter), x.dtype)
        K.quad_exp_act(up, self.pq, act)
        out = ws.get("ffn_out", (T, self.hidden_size), x.dtype)
        return matmul(act, self.w_down, None, out, target_ctas=4 * self.rt.sm_count, status=self.rt.status,
                      upcoming=ctx.upcoming)
