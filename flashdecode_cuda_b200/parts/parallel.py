"""Mixers side by side: several mixers read the same input and their outputs are added with fixed weights."""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels as K
from ..cache.paged import StateSpec
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import KVRequest, LayerCache, Mixer, Runtime
from .linear import matmul


@register_part("mixer", "parallel")
class ParallelMixers(Mixer):
    """out = sum_b scale_b * branch_b(h): ``branches`` are mixers (built parts), ``names`` what their share of the
    layer's state is called, ``scales`` their weights in the sum.

    Branches that can share their products (``shares_products``: an input product, inner work, an output product)
    are run as ONE input product over the stacked input matrices, each branch's inner work on its columns, and ONE
    output product over the branches' activations laid side by side with the stacked output matrices:
    sum_b scale_b W_b a_b = [W_1 | W_2 | ...] [scale_1 a_1 ; scale_2 a_2 ; ...].  The scale enters each branch's
    activations in float32 before their one rounding.  Other branches run whole, and the weighted sum of the outputs is
    taken in float32.  At most one branch may keep keys; every branch's per-sequence state is kept under
    ``<name>.<its own name>``."""

    def __init__(self, prefix: str, branches: Sequence[Mixer], names: Sequence[str], scales: Sequence[float],
                 hidden_size: int):
        if not branches or not (len(branches) == len(names) == len(scales)) or len(set(names)) != len(names):
            raise ValueError(f"{prefix}: branches, their names and their scales must match, names differing")
        if sum(b.kv_request() is not None for b in branches) > 1:
            raise ValueError(f"{prefix}: at most one of the mixers side by side may keep keys")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.branches, self.names, self.scales = list(branches), list(names), [float(s) for s in scales]
        self.fused = all(getattr(b, "shares_products", False) for b in self.branches)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b, "graph_safe", True) for b in self.branches)

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for b in self.branches for s in b.tensor_specs()]

    def kv_request(self) -> Optional[KVRequest]:
        for b in self.branches:
            r = b.kv_request()
            if r is not None:
                return r
        return None

    def state_requests(self) -> List[StateSpec]:
        return [StateSpec(f"{n}.{s.name}", s.shape, s.dtype) for n, b in zip(self.names, self.branches)
                for s in b.state_requests()]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        for b in self.branches:
            b.bind(tensors, rt)
        if not self.fused:
            return
        ins = [b.in_proj() for b in self.branches]
        self.w_in = torch.cat([w for w, _ in ins], dim=0).contiguous()
        self.b_in = None
        if any(bias is not None for _, bias in ins):
            self.b_in = torch.cat([bias.float() if bias is not None
                                   else torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
                                   for w, bias in ins]).contiguous()
        self.w_o = torch.cat([b.out_proj() for b in self.branches], dim=1).contiguous()
        self.in_cols, self.act_cols = [], []
        c = a = 0
        for b, (w, _) in zip(self.branches, ins):
            self.in_cols.append(c)
            self.act_cols.append(a)
            # the branch keeps views of the stacked matrices instead of copies of its own (rows of w_in are
            # contiguous; its columns of w_o are not, so alone it can no longer run)
            b.w_in = self.w_in[c:c + w.shape[0]]
            c += w.shape[0]
            a += b.out_proj().shape[1]
            b.w_o = None
            tensors.pop(f"{b.prefix}.o", None)
        self.n_act = a

    def weight_bytes(self) -> int:
        if not self.fused:
            return sum(b.weight_bytes() for b in self.branches)
        return (sum(b.weight_bytes() for b in self.branches)
                + self.w_o.numel() * self.w_o.element_size())

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_in if self.fused else self.branches[0].first_weights()

    def _sub(self, lc: LayerCache, i: int) -> LayerCache:
        pre = self.names[i] + "."
        return LayerCache(lc.group if self.branches[i].kv_request() is not None else None, lc.layer, lc.writes,
                          {k[len(pre):]: v for k, v in lc.states.items() if k.startswith(pre)})

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        if self.fused:
            proj = ws.get("par_proj", (T, self.w_in.shape[0]), x.dtype)
            matmul(x, self.w_in, self.b_in, proj, status=rt.status)
            act = ws.get("par_act", (T, self.n_act), x.dtype)
            for i, b in enumerate(self.branches):
                b.inner(ctx, proj, self.in_cols[i], self._sub(lc, i), act, self.act_cols[i], self.scales[i])
            out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
            return matmul(act, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status, upcoming=ctx.upcoming)
        total = ws.get("par_sum", (T, self.hidden_size), torch.float32)
        for i, b in enumerate(self.branches):
            y = b.forward(ctx, x, self._sub(lc, i))
            if y.dim() == 3:
                raise ValueError(f"{self.prefix}: a branch returned partial sums it was not asked for")
            K.axpy_f32(total, y, self.scales[i], accumulate=i > 0)
        return total
