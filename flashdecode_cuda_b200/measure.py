"""Measuring a model part by part: device time of every kernel launch of a step, attributed to the part that
launched it, beside the least work (floating-point operations, bytes) the part has to do.

``PartTimer(model)`` wraps, for the time it is active, the launch functions of ``kernels`` (and ``torch.mm`` /
``torch.addmm``, the library products) with CUDA events and the ``forward`` of every part with a label.  Steps must run
eagerly (``Model.step``), not from a captured graph.  The host launches far slower than the device runs a small kernel,
so the device is idle when a kernel arrives and the time between the events around a launch is that kernel's own
duration plus a launch latency of a few microseconds - the same for every model measured this way.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import kernels as K

LAUNCHERS = ["embed", "add_rmsnorm", "silu_mul", "rope_append", "gemv_qkv_rope", "gemm_tc_qkv_rope", "gemm_tc",
             "gemm_stream", "gemm_stream_qkv_rope", "gemv", "gemm_simt", "attention", "conv_rope_append",
             "conv_state_update", "gate_mul", "add_concat", "relu2", "moe_route", "moe_align", "moe_gemm", "moe_combine",
             "moe_gather", "gemm_tc_grouped", "glu_mul", "softcap", "lanes_norm", "lanes_fill", "norm_append", "head_gemm",
             "attention_ext", "attn_head_mix", "add_dyn_tanh", "quad_exp_act", "scale_", "axpy_f32", "linear_scan",
             "head_norm_gate", "add_cast", "side_gate_mul", "token_side_row", "add_row_vector", "low_rank_expand"]


class PartTimer:
    def __init__(self, model):
        self.model = model
        self.label = "other"
        self.records: List[Tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self._saved = []

    # -- wrapping ---------------------------------------------------------
    def _wrap_launcher(self, owner, name: str, shown: str) -> None:
        fn = getattr(owner, name)

        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            self.records.append((self.label, shown, e0, e1))
            return out
        self._saved.append((owner, name, fn))
        setattr(owner, name, timed)

    def _wrap_part(self, part, label: str) -> None:
        fn = part.forward

        def labelled(*a, **kw):
            before, self.label = self.label, label
            try:
                return fn(*a, **kw)
            finally:
                self.label = before
        self._saved.append((part, "forward", None))
        part.forward = labelled

    def __enter__(self) -> "PartTimer":
        for name in LAUNCHERS:
            self._wrap_launcher(K, name, name)
        self._wrap_launcher(torch, "mm", "library_mm")
        self._wrap_launcher(torch, "addmm", "library_mm")
        m = self.model
        self._wrap_part(m.embedding, "embedding")
        self._wrap_part(m.final_norm, "norm")
        self._wrap_part(m.head, "head")
        for op in m.stream_ops.values():
            self._wrap_part(op, "stream_op")
        for b in m.blocks:
            for name in ("norm1", "norm2"):
                if getattr(b, name, None) is not None:
                    self._wrap_part(getattr(b, name), "norm")
            if getattr(b, "mixer", None) is not None:
                self._wrap_part(b.mixer, "mixer")
            if getattr(b, "feed_forward", None) is not None:
                self._wrap_part(b.feed_forward, "feed_forward")
            if getattr(b, "side", None) is not None:
                self._wrap_part(b.side, "side_input")
        return self

    def __exit__(self, *exc) -> None:
        for owner, name, fn in reversed(self._saved):
            if fn is None:
                del owner.forward              # the instance attribute; the class's method shows again
            else:
                setattr(owner, name, fn)
        self._saved.clear()

    # -- results ----------------------------------------------------------
    def collect(self) -> Dict[str, Dict[str, Tuple[float, int]]]:
        """{part label: {kernel: (milliseconds in total, launches)}} of the launches recorded so far; forgets them."""
        torch.cuda.synchronize()
        out: Dict[str, Dict[str, List[float]]] = defaultdict(lambda: defaultdict(lambda: [0.0, 0]))
        for label, name, e0, e1 in self.records:
            cell = out[label][name]
            cell[0] += e0.elapsed_time(e1)
            cell[1] += 1
        self.records.clear()
        return {lab: {k: (v[0], v[1]) for k, v in d.items()} for lab, d in out.items()}


def visible_pairs(ctx_lens: Sequence[int], q_lens: Sequence[int], window: Optional[int], chunk: Optional[int],
                  keep_first: int = 0) -> int:
    """(query, key) pairs a causal attention with a window (which may keep the first positions) and / or chunks
    evaluates in a step."""
    total = 0
    for c, n in zip(ctx_lens, q_lens):
        for i in range(c, c + n):
            first = 0
            if window:
                first = max(first, i - window + 1)
            if chunk:
                first = max(first, (i // chunk) * chunk)
            total += i + 1 - first + (min(keep_first, first) if window else 0)
    return total


def keys_read(ctx_lens: Sequence[int], q_lens: Sequence[int], window: Optional[int], chunk: Optional[int],
              keep_first: int = 0) -> int:
    """Cached positions a step has to read at least once: per row, from the first key its first query sees (and the
    kept first positions)."""
    total = 0
    for c, n in zip(ctx_lens, q_lens):
        first = 0
        if window:
            first = max(first, c - window + 1)
        if chunk:
            first = max(first, (c // chunk) * chunk)
        total += c + n - first + (min(keep_first, first) if window else 0)
    return total


def part_work(part, ctx_lens: Sequence[int], q_lens: Sequence[int], real_choice_share: float = 1.0,
              experts_touched: Optional[int] = None) -> Tuple[float, float]:
    """(floating-point operations, bytes) of one run of a mixer or feed-forward over a step: products at 2 M N K,
    attention at 2 (d + dv) per pair and query head; bytes = the part's weights once (a routed feed-forward: router,
    shared expert and ``experts_touched`` experts), the cached keys and values the step has to read, and the part's
    input and output rows in the model's dtype."""
    T = sum(q_lens)
    name = type(part).__name__
    el = 2 if part.rt.dtype == torch.bfloat16 else 4
    H = part.hidden_size
    act = 2 * T * H * el
    if name == "GQAAttention":
        n_q, n_kv, d = part.n_q, part.n_kv, part.d
        pairs = visible_pairs(ctx_lens, q_lens, part.window, part.chunk)
        flops = 2 * T * H * (n_q + 2 * n_kv) * d + 2 * T * n_q * d * H + 4 * n_q * d * pairs
        kv = keys_read(ctx_lens, q_lens, part.window, part.chunk) * n_kv * 2 * d * el
        return float(flops), float(part.weight_bytes() + kv + act)
    if name == "ConvGatedAttention":
        flops, byt = _conv_attention_inner(part, ctx_lens, q_lens, el)
        n_q, dv = part.n_q, part.dv
        return float(flops + 2 * T * H * part.w_in.shape[0] + 2 * T * n_q * dv * H), float(part.weight_bytes() + byt + act)
    if name in ("Retention", "GatedLinearRecurrence"):
        flops, byt = _recurrence_inner(part, q_lens)
        nv = part.n_heads * part.dv
        return float(flops + 2 * T * H * part.w_in.shape[0] + 2 * T * nv * H), float(part.weight_bytes() + byt + act)
    if name == "ChannelDecayAttention":
        flops, byt = _recurrence_inner(part, q_lens)
        nk, nv = part.n_heads * part.d, part.n_heads * part.dv
        products = 2 * T * (H * part.w_in.shape[0] + H * part.rank + part.rank * nk + nv * H)
        return float(flops + products), float(part.weight_bytes() + byt + act)
    if name == "GatedTokenRows":
        # the stream read and written in float32, the contribution written in float32, both small matrices
        return float(2 * T * 2 * H * part.dim), float(part.weight_bytes() + 3 * T * H * 4 + T * part.dim * el)
    if name == "ParallelMixers":
        # the branches' inner work, and their input and output products once each over the stacked matrices
        flops, byt = 0.0, 0.0
        for b in part.branches:
            if type(b).__name__ == "ConvGatedAttention":
                f, y = _conv_attention_inner(b, ctx_lens, q_lens, el)
            elif type(b).__name__ in ("Retention", "GatedLinearRecurrence"):
                f, y = _recurrence_inner(b, q_lens)
            else:
                f, y = part_work(b, ctx_lens, q_lens)
                y -= act
            flops, byt = flops + f, byt + y
            if not part.fused:
                flops += 2 * T * H * (b.w_in.shape[0] + b.w_o.shape[1])
        if part.fused:
            flops += 2 * T * H * (part.w_in.shape[0] + part.w_o.shape[1])
            byt += (part.w_in.numel() + part.w_o.numel()) * el
        else:
            byt += sum(b.weight_bytes() for b in part.branches)
        return float(flops), float(byt + act)
    if name == "DenseActMLP":
        return float(2 * T * 2 * H * part.inter), float(part.weight_bytes() + act)
    if name == "QKNormedAttention":
        n_q, n_kv, d, dv = part.n_q, part.n_kv, part.d, part.dv
        pairs = visible_pairs(ctx_lens, q_lens, part.window, None)
        flops = 2 * T * H * part.w_in.shape[0] + 2 * T * n_q * dv * H + 2 * n_q * (d + dv) * pairs
        kv = keys_read(ctx_lens, q_lens, part.window, None) * n_kv * (d + dv) * el
        return float(flops), float(part.weight_bytes() + kv + act)
    if name == "LatentAttention":
        # the cheaper of attending in the latent's basis (what the part does) and expanding every visible position's
        # keys and values first (what a prompt without a cache could do)
        n_q, d, dv, r = part.n_q, part.d, part.dv, part.r
        pairs = visible_pairs(ctx_lens, q_lens, part.window, None)
        n_keys = keys_read(ctx_lens, q_lens, part.window, None)
        common = 2 * T * H * (n_q * d + r) + 2 * T * n_q * dv * H
        latent = 2 * T * n_q * r * (d + dv) + 4 * n_q * r * pairs
        expanded = 2 * n_keys * r * n_q * (d + dv) + 2 * n_q * (d + dv) * pairs
        return float(common + min(latent, expanded)), float(part.weight_bytes() + n_keys * r * el + act)
    if name in ("SwiGLU", "GatedMLP"):
        return float(2 * T * 3 * H * part.inter), float(part.weight_bytes() + act)
    if name == "RoutedExperts":
        sff = part.shared_ff or 0
        mats = 3 if getattr(part, "gated", False) else 2          # matrices of an expert
        flops = 2 * T * H * (part.E + part.n_identity) + 2 * T * part.top * real_choice_share * mats * H * part.ff \
            + 2 * T * 2 * H * sff
        touched = part.E if experts_touched is None else experts_touched
        byt = (part.E + part.n_identity) * H * el + 2 * H * sff * el + touched * mats * H * part.ff * el + act
        return float(flops), float(byt)
    raise ValueError(f"no work model for a {name}")


def _conv_attention_inner(part, ctx_lens, q_lens, el: int) -> Tuple[float, float]:
    """(operations, bytes) of a convolved attention between its two products: scores and weighted values per visible
    pair and query head, the cached keys and values the step has to read."""
    n_q, n_kv, d, dv = part.n_q, part.n_kv, part.d, part.dv
    keep = getattr(part, "keep_first", 0)
    pairs = visible_pairs(ctx_lens, q_lens, part.window, part.chunk, keep)
    kv = keys_read(ctx_lens, q_lens, part.window, part.chunk, keep) * n_kv * (d + dv) * el
    return float(2 * n_q * (d + dv) * pairs), float(kv)


def _recurrence_inner(part, q_lens) -> Tuple[float, float]:
    """(operations, bytes) of a matrix-state recurrence between its two products: per token and state element one
    multiply-add to move the state on and one to read it; every row's float32 state read and written once."""
    elements = part.n_heads * part.d * part.dv
    return float(4 * sum(q_lens) * elements), float(2 * len(q_lens) * elements * 4)


def routing_of(model, n_tokens: int, top: int, n_experts: int) -> Tuple[float, int]:
    """(share of the last routed step's choices that went to experts with weights, distinct such experts chosen),
    read from the step's workspace (the last routed layer's choices stand for all)."""
    ids = model.ws.get("moe_ids", (n_tokens, top), torch.int32).flatten().cpu()
    real = ids[ids < n_experts]
    return float(real.numel()) / max(1, ids.numel()), int(real.unique().numel())
