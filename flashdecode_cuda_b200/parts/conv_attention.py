"""Attention whose q, k and v pass through a short causal convolution over time,
with a partial rotation, chunked or windowed visibility and, by option, a sigmoid
gate on the output, biased projections, capped scores, kept first positions, a
keyless term in the softmax denominator and heads whose weights are mixed."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..cache.paged import StateSpec
from ..registry import register_part
from ..weights.spec import TensorSpec
from .attention import FP32_SPLIT_LEN, plan_splits
from .base import KVRequest, LayerCache, Mixer, Runtime
from .linear import matmul
from .normed_attention import _pad_heads, _up8


@register_part("mixer", "conv_gated_attention")
class ConvGatedAttention(Mixer):
    """For the mixer's input h [T, hidden]:

        q, k, v = W_q h, W_k h, W_v h                     (no biases)
        u_t     = sum_j c[:, j] * u_(t - taps + 1 + j)    per channel of q, k and v; zeros before the sequence
        q, k    = rotation of the first ``rot_dims`` dimensions of every head (i paired with i + rot_dims / 2,
                  angle position * base^(-2i / rot_dims)); the other dimensions pass
        a       = softmax over the visible keys of (q . k) * scale; grouped heads: query head h reads
                  key/value head h // (n_heads / n_kv_heads); value heads have ``v_head_dim`` dimensions
        out     = W_o (a * sigmoid(W_g h))                (``gate`` False: no gate)

    Visible keys of the query at position i: j <= i, of the last ``window`` positions if a window is given, and
    of i's own chunk (i // chunk == j // chunk) if a chunk is given.

    Options: ``bias`` (q, k and v have biases ``.q.b`` / ``.k.b`` / ``.v.b``, added in the projection, before the
    convolution); ``interleaved`` (the rotation pairs dimension 2i with 2i + 1 instead of i with i + rot_dims / 2);
    ``softcap`` (score <- softcap * tanh(score / softcap) after scaling); ``keep_first`` (with a window, keys at
    positions below it stay visible, at their true positions); ``sink`` (``.sink`` [heads]: exp(sink_h) is one more
    term of head h's softmax denominator, with no key and no value); ``talk`` (``.talk`` [heads, heads]: after the
    softmax the heads' weights are mixed, a'_h = sum_g talk[h, g] a_g, and head h applies a'_h to the values of its
    own key/value head).  ``sink="unit"``: the keyless term is the constant 1 (a score of zero) and has no tensor.
    ``qk_norm`` (an eps): every head of q and of k is RMS-normed over its dimensions with the weights ``.q.norm`` /
    ``.k.norm`` [head_dim], shared by the heads, after the convolution and before the rotation.  ``values_from_keys``:
    there is no value projection; a key head's values are its convolved keys as they stand before norm and rotation.
    Scores, softmax, the sink, the norms and the mixing are float32 in both dtypes.

    The last ``taps - 1`` projected values (before the convolution) of every sequence are its state, kept in
    float32 per cache slot; keys (rotated) and values (both after the convolution) go to the paged cache.
    One packed product gives q, k, v and the gate.  Tensors: ``<prefix>.q`` / ``.k`` / ``.v`` / ``.g`` / ``.o``
    (stored [out, in]) and ``<prefix>.q.conv`` / ``.k.conv`` / ``.v.conv`` ([channels, taps]).
    """

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int,
                 taps: int, scale: float, position=None, rot_dims: int = 0, chunk: Optional[int] = None,
                 window: Optional[int] = None, gate: bool = True, bias: bool = False, interleaved: bool = False,
                 softcap: Optional[float] = None, keep_first: int = 0, sink=False, talk: bool = False,
                 qk_norm: Optional[float] = None, values_from_keys: bool = False):
        for what, n in (("head size", head_dim), ("value head size", v_head_dim)):
            if n < 1 or _up8(n) > 256:
                raise ValueError(f"{prefix}: {what} {n} is not taken: the attention kernels take sizes from 1 to 256")
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0 or n_heads // n_kv_heads > 64:
            raise ValueError(f"{prefix}: {n_heads} query heads for {n_kv_heads} key/value heads: the kernels take whole "
                             f"groups of up to 64 query heads per key/value head")
        if taps < 1 or rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim or (rot_dims and position is None):
            raise ValueError(f"{prefix}: {taps} taps, {rot_dims} rotated dimensions of {head_dim}: taps must be "
                             f"positive, the rotated dimensions even, at most the head size and given a position part")
        self.prefix = prefix
        # the kernels see head sizes that are multiples of 8: other sizes are padded with zero rows of the projections,
        # biases and convolution weights (and zero columns of the output matrix) when the weights are bound, which
        # changes no score and no output
        self.d_true, self.dv_true = head_dim, v_head_dim
        self.hidden_size, self.n_q, self.n_kv, self.d, self.dv = hidden_size, n_heads, n_kv_heads, _up8(head_dim), _up8(v_head_dim)
        self.taps, self.scale, self.position, self.rot_dims = taps, float(scale), position, rot_dims
        self.chunk, self.window, self.gate = chunk, window, gate
        if softcap is not None and not softcap > 0:
            raise ValueError(f"{prefix}: the scores' soft cap must be positive, got {softcap}")
        if keep_first < 0 or (talk and gate):
            raise ValueError(f"{prefix}: keep_first must not be negative, and mixed heads take no gate")
        if sink not in (False, True, "unit"):
            raise ValueError(f"{prefix}: sink must be False, True (a learned term per head) or 'unit', got {sink!r}")
        if values_from_keys and v_head_dim != head_dim:
            raise ValueError(f"{prefix}: values taken from the keys have the keys' size {head_dim}, not {v_head_dim}")
        if qk_norm is not None and not qk_norm > 0:
            raise ValueError(f"{prefix}: the eps of the q and k norm must be positive, got {qk_norm}")
        self.bias, self.interleaved, self.softcap = bool(bias), bool(interleaved), softcap
        self.keep_first, self.sink, self.talk = int(keep_first) if window else 0, bool(sink), bool(talk)
        self.unit_sink = sink == "unit"
        self.qk_norm, self.values_from_keys = qk_norm, bool(values_from_keys)
        # the options only the CUDA-core attention kernel has
        self.extended = bool(softcap or self.keep_first or sink or talk)
        # channels that are convolved
        self.n_conv = (n_heads + n_kv_heads) * self.d + (0 if values_from_keys else n_kv_heads * self.dv)

    # --- what it needs -------------------------------------------------
    def _sizes(self):
        """(tensor, channels as stored) of the convolved projections."""
        qk = (("q", self.n_q * self.d_true), ("k", self.n_kv * self.d_true))
        return qk if self.values_from_keys else qk + (("v", self.n_kv * self.dv_true),)

    def _padded(self, name: str, t: torch.Tensor) -> torch.Tensor:
        """A tensor whose rows are the channels of q, k or v, with zero rows up to the padded head size."""
        heads, size, padded = {"q": (self.n_q, self.d_true, self.d), "k": (self.n_kv, self.d_true, self.d),
                               "v": (self.n_kv, self.dv_true, self.dv)}[name]
        return _pad_heads(t, heads, size, padded)

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        specs = []
        for n, c in self._sizes():
            specs.append(TensorSpec(f"{p}.{n}", (c, H), init="unit"))
            specs.append(TensorSpec(f"{p}.{n}.conv", (c, self.taps), "vector", init="conv"))
            if self.bias:
                specs.append(TensorSpec(f"{p}.{n}.b", (c,), "vector", init="bias"))
        if self.qk_norm is not None:
            specs += [TensorSpec(f"{p}.q.norm", (self.d_true,), "vector", init="norm"),
                      TensorSpec(f"{p}.k.norm", (self.d_true,), "vector", init="norm")]
        if self.sink and not self.unit_sink:
            specs.append(TensorSpec(f"{p}.sink", (self.n_q,), "vector", init="sink"))
        if self.talk:
            specs.append(TensorSpec(f"{p}.talk", (self.n_q, self.n_q), "vector", init="lane_mix"))
        if self.gate:
            specs.append(TensorSpec(f"{p}.g", (self.n_q * self.dv_true, H), init="unit"))
        specs.append(TensorSpec(f"{p}.o", (H, self.n_q * self.dv_true), init="unit"))
        return specs

    def kv_request(self) -> KVRequest:
        return KVRequest(self.n_kv, self.d, self.window, self.chunk, self.dv, keep_first=self.keep_first)

    def state_requests(self) -> List[StateSpec]:
        if self.taps == 1:
            return []
        return [StateSpec("conv", (self.taps - 1, self.n_conv), torch.float32)]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        mats = [self._padded(n, tensors.pop(f"{p}.{n}")) for n, _ in self._sizes()]
        if self.gate:
            mats.append(_pad_heads(tensors.pop(f"{p}.g"), self.n_q, self.dv_true, self.dv))
        self.w_in = torch.cat(mats, dim=0).contiguous()            # [q | k | v | gate] rows: one product
        self.b_in = None
        if self.bias:
            b = [self._padded(n, tensors.pop(f"{p}.{n}.b").float()) for n, _ in self._sizes()]
            if self.gate:
                b.append(torch.zeros(self.n_q * self.dv, dtype=torch.float32, device=b[0].device))
            self.b_in = torch.cat(b).contiguous()
        self.conv_w = torch.cat([self._padded(n, tensors.pop(f"{p}.{n}.conv").float()) for n, _ in self._sizes()],
                                dim=0).contiguous()
        self.sink_w = None
        if self.unit_sink:
            self.sink_w = torch.zeros(self.n_q, dtype=torch.float32, device=rt.device)
        elif self.sink:
            self.sink_w = tensors.pop(f"{p}.sink").float().contiguous()
        self.q_norm_w = self.k_norm_w = None
        if self.qk_norm is not None:         # zero weights on the padded dimensions; the mean runs over the true ones
            self.q_norm_w = _pad_heads(tensors.pop(f"{p}.q.norm").float(), 1, self.d_true, self.d).contiguous()
            self.k_norm_w = _pad_heads(tensors.pop(f"{p}.k.norm").float(), 1, self.d_true, self.d).contiguous()
        self.talk_w = tensors.pop(f"{p}.talk").float().contiguous() if self.talk else None
        self.w_o = tensors[f"{p}.o"]
        if self.dv != self.dv_true:         # zero columns where the padded value dimensions arrive
            self.w_o = _pad_heads(tensors.pop(f"{p}.o").t().contiguous(), self.n_q, self.dv_true, self.dv).t().contiguous()

    def weight_bytes(self) -> int:
        w_o = self.w_o.numel() * self.w_o.element_size() if self.w_o is not None else 0
        return self.w_in.numel() * self.w_in.element_size() + w_o + self.conv_w.numel() * 4

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_in

    # --- as one of several mixers that share their input and output products (``parts.parallel``) ------------
    @property
    def shares_products(self) -> bool:
        """Whether ``inner`` can leave its activations, scaled, in a column range of a wider buffer: with mixed
        heads the mixing kernel is the one that writes them."""
        return self.talk

    def in_proj(self):
        return self.w_in, self.b_in

    def out_proj(self) -> torch.Tensor:
        return self.w_o

    # --- a step ----------------------------------------------------------
    def inner(self, ctx, proj: torch.Tensor, col0: int, lc: LayerCache, act: Optional[torch.Tensor] = None,
              act_col: int = 0, scale: float = 1.0) -> torch.Tensor:
        """From this mixer's columns of ``proj`` (starting at ``col0``) to the input of its output product.  With
        ``act`` given (mixed heads only) that is written, times ``scale``, into act[:, act_col:]; else returned."""
        T, ws, rt = ctx.T, ctx.ws, self.rt
        dt = proj.dtype
        q = ws.get("cga_q", (T, self.n_q * self.d), dt)
        state = lc.states.get("conv")
        rope = self.position
        single = ctx.max_q_len == 1                     # every row brings one token: the state moves on in the same kernel
        K.conv_rope_append(proj, self.conv_w, state, q, rope.cos if self.rot_dims else None,
                           rope.sin if self.rot_dims else None, self.rot_dims, ctx.tok_row, ctx.tok_pos, ctx.row_slot,
                           ctx.row_q_start, ctx.row_q_len, lc.k_pool, lc.v_pool, lc.group.table, self.n_q, self.n_kv,
                           self.d, self.dv, lc.writes, single and lc.writes, rt.status, interleaved=self.interleaved,
                           first_col=col0, q_norm=self.q_norm_w, k_norm=self.k_norm_w, norm_eps=self.qk_norm or 0.0,
                           norm_count=self.d_true, values_from_keys=self.values_from_keys)
        if state is not None and lc.writes and not single:
            K.conv_state_update(proj, state, ctx.row_slot, ctx.row_q_start, ctx.row_q_len, ctx.n_rows, first_col=col0)
        heads_out = self.n_q * (self.n_kv if self.talk else 1)      # mixed heads: every head's weights on every value head
        n_splits, split_len, scratch = 1, 0, None
        if single:
            if dt == torch.float32:
                # splits of a fixed length: where a sequence's partial sums are cut depends on its own length only
                split_len = FP32_SPLIT_LEN
                n_splits = max(1, -(-ctx.kv_len_bound // split_len))
            else:
                # CTAs per sequence and split: one per key head and value head it meets, or - mixed heads of up to 64
                # query rows in all - one per key head, which takes all value heads
                per_seq = self.n_kv if self.talk and self.n_q <= 64 else heads_out // (self.n_q // self.n_kv)
                # with a window only its keys and the kept ones are read: the splits are sized for those, so that the
                # CTAs that find keys are about as many as the SMs, and laid over the whole length
                seen = ctx.kv_len_bound
                if self.window:
                    seen = min(seen, self.window + self.keep_first + 32)
                _, split_len = plan_splits(ctx.n_rows, per_seq, seen, rt.sm_count)
                n_splits = max(1, -(-ctx.kv_len_bound // split_len))
                if n_splits > 64:                       # bounded scratch memory and merge
                    split_len = -(-(-(-ctx.kv_len_bound // 64)) // 32) * 32
                    n_splits = -(-ctx.kv_len_bound // split_len)
            if n_splits > 1:
                scratch = ws.get("attn_scratch", (K.attention_scratch_floats(T, heads_out, self.dv, n_splits),),
                                 torch.float32)
        if not self.extended:
            attn = ws.get("cga_attn", (T, self.n_q * self.dv), dt)
            K.attention(q, lc.k_pool, lc.v_pool, attn, lc.group.table, ctx.tok_row, ctx.row_slot, ctx.row_q_start,
                        ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, ctx.max_q_len, self.n_q, self.n_kv, self.d, self.scale,
                        self.window or 0, n_splits, split_len, scratch, rt.status, chunk=self.chunk or 0)
        else:
            attn = ws.get("cga_attn_f" if self.talk else "cga_attn", (T, heads_out * self.dv),
                          torch.float32 if self.talk else dt)
            K.attention_ext(q, lc.k_pool, lc.v_pool, attn, lc.group.table, ctx.tok_row, ctx.row_slot, ctx.row_q_start,
                            ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, ctx.max_q_len, self.n_q, self.n_kv, self.d,
                            self.scale, self.window or 0, n_splits, split_len, scratch, rt.status, chunk=self.chunk or 0,
                            softcap=self.softcap or 0.0, keep_first=self.keep_first, sink=self.sink_w,
                            all_value_heads=self.talk)
        if self.talk:
            if act is None:
                act, act_col = ws.get("cga_mixed", (T, self.n_q * self.dv), dt), 0
            K.attn_head_mix(attn, self.talk_w, act, act_col, self.n_q, self.n_kv, self.dv, scale)
            return act
        if act is not None:
            raise ValueError(f"{self.prefix}: without mixed heads this mixer keeps its own output product")
        if self.gate:
            gated = ws.get("cga_gated", (T, self.n_q * self.dv), dt)
            K.gate_mul(attn, proj, col0 + self.n_conv, gated)
            attn = gated
        return attn

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        proj = ws.get("cga_proj", (T, self.w_in.shape[0]), x.dtype)
        matmul(x, self.w_in, self.b_in, proj, status=rt.status)
        attn = self.inner(ctx, proj, 0, lc)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        return matmul(attn, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status)
