"""Mixers that carry a matrix state per head instead of keys: linear attention with a constant decay per head
(retention) and with a forget gate per channel that also decides what is written (a gated linear recurrence)."""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels as K
from ..cache.paged import StateSpec
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import LayerCache, Mixer, Runtime
from .linear import matmul


class _StateMixer(Mixer):
    """What the two recurrences share: a state [heads, head_dim, v_head_dim] in float32 per cache slot, one packed
    input product, and the protocol by which several mixers share their input and output products."""

    shares_products = True

    def kv_request(self):
        return None

    def state_requests(self) -> List[StateSpec]:
        return [StateSpec("state", (self.n_heads, self.d, self.dv), torch.float32)]

    def weight_bytes(self) -> int:
        w_o = self.w_o.numel() * self.w_o.element_size() if self.w_o is not None else 0
        return self.w_in.numel() * self.w_in.element_size() + w_o

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_in

    def in_proj(self):
        return self.w_in, self.b_in

    def out_proj(self) -> torch.Tensor:
        return self.w_o

    def scan_scratch(self, ctx) -> Optional[torch.Tensor]:
        """Scratch memory for a step with a portion long enough to run in segments; None for the others."""
        if ctx.max_q_len <= 2 * K.linear_scan_segment():
            return None
        n = K.linear_scan_scratch_floats(ctx.T, ctx.n_rows, self.n_heads, self.d, self.dv)
        return ctx.ws.get("scan_segments", (n,), torch.float32)

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        proj = ws.get("rec_proj", (T, self.w_in.shape[0]), x.dtype)
        matmul(x, self.w_in, self.b_in, proj, status=rt.status)
        act = ws.get("rec_act", (T, self.n_heads * self.dv), x.dtype)
        self.inner(ctx, proj, 0, lc, act, 0, 1.0)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        return matmul(act, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status, upcoming=ctx.upcoming)


@register_part("mixer", "retention")
class Retention(_StateMixer):
    """For the mixer's input h [T, hidden], per head with the constant decay g_h:

        q, k = rot(W_q h), rot(W_k h) * head_dim^(-1/2);  v = W_v h          (no biases)
        S_t  = g_h S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t                  (no softmax, no denominator)
        out  = W_o ( concat_h o_t / rms(o_t) * silu(W_g h) )               (rms over a head's ``v_head_dim``, with eps)

    rot turns the first ``rot_dims`` dimensions of every head at the token's position, dimension i paired with
    i + rot_dims / 2.  The state starts at zero and is carried in float32 per cache slot; rotation, decay, state,
    output and the norm are float32 in both dtypes.  Tensors ``<prefix>.q`` / ``.k`` / ``.v`` / ``.g`` / ``.o``."""

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, head_dim: int, v_head_dim: int,
                 decay: Sequence[float], eps: float, position=None, rot_dims: int = 0):
        if len(decay) != n_heads:
            raise ValueError(f"{prefix}: {len(decay)} decays for {n_heads} heads")
        if head_dim > 256 or min(n_heads, head_dim, v_head_dim) < 1:
            raise ValueError(f"{prefix}: heads of {head_dim} x {v_head_dim}: the recurrence takes key sizes up to 256")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim or (rot_dims and position is None):
            raise ValueError(f"{prefix}: {rot_dims} rotated dimensions of {head_dim}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.n_heads, self.d, self.dv = n_heads, head_dim, v_head_dim
        self.decay, self.eps, self.position, self.rot_dims = [float(g) for g in decay], float(eps), position, rot_dims

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        return [TensorSpec(f"{p}.q", (nk, H), init="unit"), TensorSpec(f"{p}.k", (nk, H), init="unit"),
                TensorSpec(f"{p}.v", (nv, H), init="unit"), TensorSpec(f"{p}.g", (nv, H), init="unit"),
                TensorSpec(f"{p}.o", (H, nv), init="unit")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        self.w_in = torch.cat([tensors.pop(f"{p}.{n}") for n in "qkvg"], dim=0).contiguous()
        self.b_in = None
        self.w_o = tensors[f"{p}.o"]
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)

    def inner(self, ctx, proj: torch.Tensor, col0: int, lc: LayerCache, act: torch.Tensor, act_col: int = 0,
              scale: float = 1.0) -> torch.Tensor:
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        o = ctx.ws.get("scan_out", (ctx.T, nv), torch.float32)
        rope = self.position
        K.linear_scan(proj, col0, col0 + nk, col0 + 2 * nk, lc.states["state"], o, K.SCAN_DECAY, ctx.row_slot,
                      ctx.row_q_start, ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, self.n_heads, self.d, self.dv,
                      lc.writes, self.rt.status, decay=self.decay_dev, cos=rope.cos if self.rot_dims else None,
                      sin=rope.sin if self.rot_dims else None, rot_dims=self.rot_dims, k_scale=self.d ** -0.5,
                      max_q_len=ctx.max_q_len, scratch=self.scan_scratch(ctx))
        K.head_norm_gate(o, act, act_col, self.n_heads, self.dv, self.eps, None, proj, col0 + 2 * nk + nv, scale)
        return act


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(_StateMixer):
    """For the mixer's input h [T, hidden], per head:

        q = silu(W_q h);  v = W_v h;  f = lower + (1 - lower) * sigmoid(W_f h + b_f)     (per channel of q)
        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;   o_t = S_t^T q_t                     (no key, no other scale)
        out = W_o ( concat_h o_t / rms(o_t) * w )                                        (w [v_head_dim], shared by heads)

    The state starts at zero and is carried in float32 per cache slot; gate, state, output and the norm are float32 in
    both dtypes.  Tensors ``<prefix>.q`` / ``.f`` / ``.f.b`` / ``.lower`` / ``.v`` / ``.norm`` / ``.o``."""

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, head_dim: int, v_head_dim: int, eps: float):
        if head_dim > 256 or min(n_heads, head_dim, v_head_dim) < 1:
            raise ValueError(f"{prefix}: heads of {head_dim} x {v_head_dim}: the recurrence takes key sizes up to 256")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.n_heads, self.d, self.dv, self.eps = n_heads, head_dim, v_head_dim, float(eps)

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        return [TensorSpec(f"{p}.q", (nk, H), init="unit"), TensorSpec(f"{p}.f", (nk, H), init="unit"),
                TensorSpec(f"{p}.f.b", (nk,), "vector", init="bias"),
                TensorSpec(f"{p}.lower", (nk,), "vector", init="unit_interval"),
                TensorSpec(f"{p}.v", (nv, H), init="unit"), TensorSpec(f"{p}.norm", (self.dv,), "vector", init="norm"),
                TensorSpec(f"{p}.o", (H, nv), init="unit")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        self.w_in = torch.cat([tensors.pop(f"{p}.{n}") for n in "qfv"], dim=0).contiguous()
        fb = tensors.pop(f"{p}.f.b").float()
        self.b_in = torch.cat([torch.zeros(nk, dtype=torch.float32, device=fb.device), fb,
                               torch.zeros(nv, dtype=torch.float32, device=fb.device)]).contiguous()
        self.lower = tensors.pop(f"{p}.lower").float().contiguous()
        self.norm_w = tensors.pop(f"{p}.norm").float().contiguous()
        self.w_o = tensors[f"{p}.o"]

    def inner(self, ctx, proj: torch.Tensor, col0: int, lc: LayerCache, act: torch.Tensor, act_col: int = 0,
              scale: float = 1.0) -> torch.Tensor:
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        o = ctx.ws.get("scan_out", (ctx.T, nv), torch.float32)
        K.linear_scan(proj, col0, col0 + nk, col0 + 2 * nk, lc.states["state"], o, K.SCAN_GATED, ctx.row_slot,
                      ctx.row_q_start, ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, self.n_heads, self.d, self.dv,
                      lc.writes, self.rt.status, lower=self.lower, max_q_len=ctx.max_q_len, scratch=self.scan_scratch(ctx))
        K.head_norm_gate(o, act, act_col, self.n_heads, self.dv, self.eps, self.norm_w, None, 0, scale)
        return act


@register_part("mixer", "channel_decay_attention")
class ChannelDecayAttention(_StateMixer):
    """Linear attention with a decay per key channel that follows the input.  For the mixer's input h [T, hidden], per
    head:

        q = W_q h * head_dim^(-1/2);  k = W_k h;  v = W_v h                           (no biases)
        a = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)                                   per channel of k, through a narrow W_a1
        S_t = diag(a_t) S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t
        out = W_o ( concat_h o_t / rms(o_t) * w * silu(W_g h) )                       (w [v_head_dim], shared by heads)

    The state starts at zero and is carried in float32 per cache slot.  W_a1 of up to 64 rows rides in the packed input
    product and one kernel expands its output to the channels (``low_rank_expand``); the decay's pre-activation is
    float32 either way, and the sigmoid, its logarithm, the power, the state, the output and the norm are float32 in both dtypes.
    Tensors ``<prefix>.q`` / ``.k`` / ``.v`` / ``.g`` / ``.o`` / ``.norm`` / ``.a1`` / ``.a2`` / ``.a2.b``.
    ``decay_rank`` (the rows of W_a1) None: the checkpoint's tensors give it."""

    shares_products = False

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, head_dim: int, v_head_dim: int,
                 tau: float, eps: float, decay_rank: Optional[int] = None):
        if head_dim > 256 or min(n_heads, head_dim, v_head_dim, 1 if decay_rank is None else decay_rank) < 1:
            raise ValueError(f"{prefix}: heads of {head_dim} x {v_head_dim}: the recurrence takes key sizes up to 256")
        if not tau > 0:
            raise ValueError(f"{prefix}: the decay's temperature must be positive, got {tau}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.n_heads, self.d, self.dv, self.rank = n_heads, head_dim, v_head_dim, decay_rank
        self.tau, self.eps = float(tau), float(eps)

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        return [TensorSpec(f"{p}.q", (nk, H), init="unit"), TensorSpec(f"{p}.k", (nk, H), init="unit"),
                TensorSpec(f"{p}.v", (nv, H), init="unit"), TensorSpec(f"{p}.g", (nv, H), init="unit"),
                TensorSpec(f"{p}.o", (H, nv), init="unit"), TensorSpec(f"{p}.norm", (self.dv,), "vector", init="norm"),
                TensorSpec(f"{p}.a1", (self.rank, H), init="unit"), TensorSpec(f"{p}.a2", (nk, self.rank), init="unit"),
                TensorSpec(f"{p}.a2.b", (nk,), "vector", init="decay_bias")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        self.w_a1, self.w_a2 = tensors[f"{p}.a1"], tensors[f"{p}.a2"]
        if self.w_a1.shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"{p}: a1 has {self.w_a1.shape[0]} rows and a2 {self.w_a2.shape[1]} columns")
        self.rank = self.w_a1.shape[0]
        # a narrow projection rides in the packed input product, and one kernel expands it to the channels; a wide one
        # keeps two products of its own
        self.packed_decay = self.rank <= K.LOW_RANK_EXPAND_MAX
        mats = [tensors.pop(f"{p}.{n}") for n in "qkvg"] + ([self.w_a1] if self.packed_decay else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.b_in = None
        self.b_a2 = tensors.pop(f"{p}.a2.b").float().contiguous()
        self.norm_w = tensors.pop(f"{p}.norm").float().contiguous()
        self.w_o = tensors[f"{p}.o"]

    def weight_bytes(self) -> int:
        own = 0 if self.packed_decay else self.w_a1.numel() * self.w_a1.element_size()
        return super().weight_bytes() + own + self.w_a2.numel() * self.w_a2.element_size()

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        nk, nv = self.n_heads * self.d, self.n_heads * self.dv
        proj = ws.get("rec_proj", (T, self.w_in.shape[0]), x.dtype)
        matmul(x, self.w_in, None, proj, status=rt.status)
        z = ws.get("rec_decay_z", (T, nk), torch.float32)
        if self.packed_decay:
            K.low_rank_expand(proj, 2 * nk + 2 * nv, self.w_a2, self.b_a2, z)
        else:
            low = ws.get("rec_decay_low", (T, self.rank), x.dtype)
            matmul(x, self.w_a1, None, low, status=rt.status)
            matmul(low, self.w_a2, self.b_a2, z, status=rt.status)
        o = ws.get("scan_out", (T, nv), torch.float32)
        K.linear_scan(proj, 0, nk, 2 * nk, lc.states["state"], o, K.SCAN_CHANNEL_DECAY, ctx.row_slot, ctx.row_q_start,
                      ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, self.n_heads, self.d, self.dv, lc.writes, rt.status,
                      max_q_len=ctx.max_q_len, scratch=self.scan_scratch(ctx), gate=z, q_scale=self.d ** -0.5, tau=self.tau)
        act = ws.get("rec_act", (T, nv), x.dtype)
        K.head_norm_gate(o, act, 0, self.n_heads, self.dv, self.eps, self.norm_w, proj, 2 * nk + nv, 1.0)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        return matmul(act, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status, upcoming=ctx.upcoming)
