"""Routed feed-forward: a mixture of small experts chosen per token."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime
from .linear import fused_prompt_gemm, matmul

# Up to this many tokens the routing kernel makes the router's logits itself (one launch, a CTA per token, each reading
# the whole router matrix); above it they come from a matrix product.
ROUTE_FUSED_MAX_TOKENS = 64
# ... and up to this many router weights: every token's CTA reads the whole matrix, a chain of latencies that a
# weight-streaming product spread over the GPU does not have (64 outputs at width 2,048, batch 8: the routing kernel 18 us
# on its own, 7 with the logits from the product; the decode step 0.878 -> 0.849 ms; 16 outputs at width 1,024: no difference)
ROUTE_FUSED_MAX_WEIGHTS = 65536
# Which kernel takes the grouped products of steps with many rows per expert in bfloat16: "auto": the TMA + tcgen05
# kernel where it takes the sizes (expert matrices of at least 256 rows), else the mma.sync kernel; "mma": the
# mma.sync kernel always (tests run both).
GROUPED_GEMM = "auto"


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """For the feed-forward's input h [T, hidden]:

        s      = softmax(W_router h) over all ``n_experts + n_identity`` router outputs   (float32)
        chosen = the ``top`` outputs with the largest s + correction
        w      = s[chosen] / (sum of s[chosen] + 1e-20)
        out    = sum over chosen e of w_e * expert_e(h)  +  shared(h)

    An expert, and the shared expert, is down(act(up h)) with act = relu^2 and no biases; with ``expert_act =
    "clamped_swish"`` an expert is gated instead: g = min(gate h, limit), u = clamp(up h, -limit, limit),
    down(g sigmoid(1.702 g) (u + 1)) (tensors ``.e<i>.gate`` too).  ``router_bias``: ``<prefix>.router.b`` is added to
    the router's outputs before the softmax; w is then the softmax over the chosen outputs alone.  The last
    ``n_identity`` router outputs are identity experts: they have no tensors and pass h on.  ``shared_ff``
    None: no shared expert.  ``expert_act = "silu_gated"``: an expert is down(silu(gate h) * (up h)).
    ``score = "sigmoid"``: s = sigmoid(W_router h), each output by itself.  ``groups = (count, keep)``: the router's
    outputs form ``count`` equal groups of neighbours; a group ranks by the sum of its two largest s + correction, and
    only outputs of the best ``keep`` groups can be chosen.  ``weight_scale``: w = s[chosen] * weight_scale, not
    divided by the chosen scores' sum.

    All decisions are taken on the device (no read-back): the (token, choice) pairs are grouped by expert, each
    group padded to whole row tiles, and two grouped products run over the tiles that exist.  Tensors:
    ``<prefix>.e<i>.up`` [ff, hidden], ``<prefix>.e<i>.down`` [hidden, ff], ``<prefix>.router``,
    ``<prefix>.correction``, ``<prefix>.shared.up`` / ``.down``.
    """

    def __init__(self, prefix: str, hidden_size: int, n_experts: int, top: int, expert_ff: int, n_identity: int = 0,
                 shared_ff: Optional[int] = None, correction: bool = True, expert_act: str = "relu2",
                 limit: Optional[float] = None, router_bias: bool = False, score: str = "softmax",
                 groups: Optional[tuple] = None, weight_scale: Optional[float] = None):
        if n_experts < 0 or n_identity < 0 or not (1 <= top <= n_experts + n_identity) or expert_ff < 1:
            raise ValueError(f"{prefix}: {top} choices among {n_experts} experts and {n_identity} identity experts")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.E, self.n_identity, self.top, self.ff, self.shared_ff = n_experts, n_identity, top, expert_ff, shared_ff
        self.has_correction = correction
        if expert_act not in ("relu2", "clamped_swish", "silu_gated") or (expert_act == "clamped_swish" and not (limit and limit > 0)):
            raise ValueError(f"{prefix}: expert activation {expert_act!r} (relu2, silu_gated, or clamped_swish with a positive limit)")
        self.gated, self.router_bias = expert_act in ("clamped_swish", "silu_gated"), bool(router_bias)
        self.limit = limit if expert_act == "clamped_swish" else None
        self.glu_kind = K.GLU_CLAMPED if expert_act == "clamped_swish" else K.GLU_SILU
        # how the grouped products' gated epilogues are told the activation
        self.gated_args = dict(gated_limit=limit) if expert_act == "clamped_swish" else dict(gated_act=K.GLU_SILU)
        if score not in ("softmax", "sigmoid"):
            raise ValueError(f"{prefix}: router scores {score!r} (softmax or sigmoid)")
        self.sigmoid_scores = score == "sigmoid"
        n_out = n_experts + n_identity
        self.n_groups, self.keep_groups = (1, 1) if not groups else (int(groups[0]), int(groups[1]))
        if (self.n_groups < 1 or n_out % self.n_groups or not (1 <= self.keep_groups <= self.n_groups)
                or self.keep_groups * (n_out // self.n_groups) < top):
            raise ValueError(f"{prefix}: {self.keep_groups} of {self.n_groups} groups of {n_out} router outputs for "
                             f"{top} choices: the groups must be equal and the kept ones hold enough outputs")
        self.weight_scale = None if weight_scale is None else float(weight_scale)

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        specs = []
        for e in range(self.E):
            if self.gated:
                specs.append(TensorSpec(f"{p}.e{e}.gate", (self.ff, H), init="unit"))
            specs += [TensorSpec(f"{p}.e{e}.up", (self.ff, H), init="unit"),
                      TensorSpec(f"{p}.e{e}.down", (H, self.ff), init="unit")]
        specs.append(TensorSpec(f"{p}.router", (self.E + self.n_identity, H), init="unit"))
        if self.router_bias:
            specs.append(TensorSpec(f"{p}.router.b", (self.E + self.n_identity,), "vector", init="bias"))
        if self.has_correction:
            specs.append(TensorSpec(f"{p}.correction", (self.E + self.n_identity,), "vector", init="bias"))
        if self.shared_ff is not None:
            specs += [TensorSpec(f"{p}.shared.up", (self.shared_ff, H), init="unit"),
                      TensorSpec(f"{p}.shared.down", (H, self.shared_ff), init="unit")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        if self.E:
            if self.gated:
                # [E, 2 ff, H]: one product for an expert's gate and up rows.  bfloat16: in tiles of 8 gate rows + the 8 up
                # rows of the same outputs, for the products' gated epilogues; float32: gate rows, then up rows
                self.tiled = rt.dtype == torch.bfloat16 and self.ff % 8 == 0
                f8 = self.ff // 8

                def pack(g, u):
                    if not self.tiled:
                        return torch.cat([g, u])
                    return torch.stack([g.view(f8, 8, -1), u.view(f8, 8, -1)], dim=1).reshape(2 * self.ff, -1)
                self.w_up = torch.stack([pack(tensors.pop(f"{p}.e{e}.gate"), tensors.pop(f"{p}.e{e}.up"))
                                         for e in range(self.E)]).contiguous()
            else:
                self.w_up = torch.stack([tensors.pop(f"{p}.e{e}.up") for e in range(self.E)]).contiguous()   # [E, ff, H]
            self.w_down = torch.stack([tensors.pop(f"{p}.e{e}.down") for e in range(self.E)]).contiguous()   # [E, H, ff]
        else:
            self.w_up = self.w_down = None
        self.router = tensors[f"{p}.router"]
        self.correction = tensors[f"{p}.correction"].float().contiguous() if self.has_correction else None
        self.r_bias = tensors[f"{p}.router.b"].float().contiguous() if self.router_bias else None
        self.s_up = tensors.get(f"{p}.shared.up")
        self.s_down = tensors.get(f"{p}.shared.down")

    def weight_bytes(self) -> int:
        """What a step reads at most: every expert once (a decode step of few tokens reads only the chosen ones)."""
        n = self.router.numel() * self.router.element_size()
        for w in (self.w_up, self.w_down, self.s_up, self.s_down):
            if w is not None:
                n += w.numel() * w.element_size()
        return n

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.s_up if self.s_up is not None else self.router

    def _shared_expert(self, ctx, x: torch.Tensor) -> torch.Tensor:
        T, ws, H = ctx.T, ctx.ws, self.hidden_size
        h = ws.get("moe_shared_h", (T, self.shared_ff), x.dtype)
        if x.dtype == torch.bfloat16 and fused_prompt_gemm(T, self.shared_ff, H):
            K.gemm_tc(x, self.s_up, None, h, status=self.rt.status, relu2=True)      # prompts: the activation in the epilogue
        else:
            matmul(x, self.s_up, None, h, status=self.rt.status)
            K.relu2(h, h)
        shared = ws.get("moe_shared_out", (T, H), x.dtype)
        return matmul(h, self.s_down, None, shared, target_ctas=4 * self.rt.sm_count, status=self.rt.status)

    def forward(self, ctx, x: torch.Tensor, parts_ok: bool = False) -> torch.Tensor:
        T, ws, H, top = ctx.T, ctx.ws, self.hidden_size, self.top
        # the shared expert depends on nothing of the routing.  (On a second stream beside the routed experts it gained
        # 4 % in a 2,048-token prompt step at width 2,048, lost 10 % at width 1,024, where the host sets the pace, and
        # changed nothing in captured decode steps, whose kernels each fill the GPU: it runs in line.)
        shared = self._shared_expert(ctx, x) if self.s_up is not None else None
        ids = ws.get("moe_ids", (T, top), torch.int32)
        wts = ws.get("moe_wts", (T, top), torch.float32)
        logits = None
        if (x.dtype == torch.float32 or T > ROUTE_FUSED_MAX_TOKENS or H > K.ROUTE_FUSED_MAX_ROW
                or self.router.numel() > ROUTE_FUSED_MAX_WEIGHTS):
            # many tokens: the logits as one product (float32 out: bfloat16 operands multiply exactly, sums are float).
            # float32 always takes this way: its product sums k in one fixed order whatever the step holds, so a
            # token's scores do not change by a bit with its neighbours
            logits = ws.get("moe_logits", (T, self.router.shape[0]), torch.float32)
            matmul(x, self.router, None, logits, status=self.rt.status)
        K.moe_route(x, self.router, self.correction, ids, wts, logits, bias=self.r_bias,
                    sigmoid_scores=self.sigmoid_scores, n_groups=self.n_groups, keep_groups=self.keep_groups,
                    weight_scale=self.weight_scale)
        # (the routed experts follow on the main stream; the shared expert's stream joins before the combine)
        y = pair_pos = None
        pair_pos = ws.get("moe_pair_pos", (T * top,), torch.int32)
        if self.E:
            mt = K.moe_tile_rows(x.dtype, T * top, self.E, (H, self.ff))
            cap = K.moe_grouped_rows(T * top, self.E, mt)
            sorted_pair = ws.get("moe_sorted", (cap,), torch.int32)
            tile_expert = ws.get("moe_tile_expert", (cap // mt,), torch.int32)
            n_tiles = ws.get("moe_n_tiles", (1,), torch.int32)
            K.moe_align(ids, self.E, pair_pos, sorted_pair, tile_expert, n_tiles, mt)
            act = ws.get("moe_act", (cap, self.ff), x.dtype)
            y = ws.get("moe_y", (cap, H), x.dtype)
            n_up = self.w_up.shape[1]                   # ff, or 2 ff for gated experts
            fused = self.gated and self.tiled           # the gated activation in the up product's epilogue
            gu = ws.get("moe_gu", (cap, n_up), x.dtype) if self.gated and not fused else None
            if (mt == 128 and GROUPED_GEMM == "auto" and K.gemm_tc_grouped_supported(n_up, H)
                    and K.gemm_tc_grouped_supported(H, self.ff)):
                # prompts: the grouped rows as one matrix, then both products on the tcgen05 tensor cores
                xs = ws.get("moe_xs", (cap, H), x.dtype)
                K.moe_gather(x, xs, sorted_pair, n_tiles, top, mt)
                if fused and n_up % 32 == 0:
                    K.gemm_tc_grouped(xs, self.w_up, act, False, tile_expert, n_tiles, self.rt.status, **self.gated_args)
                elif self.gated:
                    gu = ws.get("moe_gu", (cap, n_up), x.dtype)
                    K.gemm_tc_grouped(xs, self.w_up, gu, False, tile_expert, n_tiles, self.rt.status)
                    K.glu_mul(gu, act, self.glu_kind, self.limit or 0.0, tiled=self.tiled)
                else:
                    K.gemm_tc_grouped(xs, self.w_up, act, True, tile_expert, n_tiles, self.rt.status)
                K.gemm_tc_grouped(act, self.w_down, y, False, tile_expert, n_tiles, self.rt.status)
            else:
                if fused:
                    K.moe_gemm(x, self.w_up, act, False, sorted_pair, tile_expert, n_tiles, top, mt, **self.gated_args)
                elif self.gated:
                    K.moe_gemm(x, self.w_up, gu, False, sorted_pair, tile_expert, n_tiles, top, mt, plain=True)
                    K.glu_mul(gu, act, self.glu_kind, self.limit or 0.0)
                else:
                    K.moe_gemm(x, self.w_up, act, False, sorted_pair, tile_expert, n_tiles, top, mt)
                K.moe_gemm(act, self.w_down, y, True, sorted_pair, tile_expert, n_tiles, top, mt)
        out = ws.get("ffn_out", (T, H), x.dtype)
        K.moe_combine(y, x, shared, ids, wts, pair_pos, out, self.E)
        return out
