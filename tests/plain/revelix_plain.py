"""Plain, slow implementation of the Revelix decoder: whole sequences, no cache,
one function per mechanism.  It shares no code with the product package; it
reads a raw ``config.json`` dictionary and a ``{tensor name: tensor}`` dict.

Revelix in this file's notation.  A layer is pre-norm, x += mixer(n1(x)) and, if
the layer has a feed-forward, x += ff(n2(x)); n(x) = tanh(alpha x) * w + b with a
scalar alpha (no mean, no variance).  Two kinds of mixer:

* ``retention``: linear attention with a constant decay g_h per head,
  S_t = g_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q and k are rotated (pairs
  (i, i + dims/2)) and k is scaled by dim^(-1/2); every head's output is divided
  by its root mean square, the heads are multiplied by silu(W_g h) and projected.
* ``parallel``: the weighted sum of two branches on the same input.  The left
  branch is grouped-head softmax attention with biased projections, a short
  causal convolution on q, k and v, a rotation of interleaved pairs (2i, 2i+1)
  with stretched frequencies, tanh-capped scores, a window that also keeps the
  first positions, one extra learned term per head in the softmax denominator,
  and a matrix that mixes the heads' weights after the softmax.  The right
  branch is a gated linear recurrence S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T
  read by q_t = silu(W_q h_t), with a lower-bounded forget gate f and a weighted
  RMS norm per head.

The feed-forward is W_down a(W_up h) with a two-parameter activation that is
quadratic above zero and exponential below.  The logits are the final norm's
output times the embedding table, times a constant.

The arithmetic dtype is a parameter (float64 by default).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def dyn_tanh(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    return torch.tanh(alpha * x) * w + b


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rot_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """(frequencies [dims/2], factor on cos and sin).  Without ``scaling``: base^(-2i/dims) and 1.  With it, the
    frequencies of slowly turning pairs are divided by ``factor``, fast ones kept, with a linear ramp between the pair
    indices at which ``original`` positions hold ``fast`` and ``slow`` turns; cos and sin grow by 0.1 ln(factor) + 1."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, freqs: torch.Tensor, mag: float,
           interleaved: bool) -> torch.Tensor:
    """x [S, heads, d]: the first ``dims`` dimensions of each head are rotated by position * freqs; pair i is
    (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``.  (u, v) -> (u c - v s, v c + u s), c and s times ``mag``."""
    a = positions.to(torch.float64)[:, None] * freqs[None, :]
    c, s = (torch.cos(a) * mag).to(x.dtype)[:, None, :], (torch.sin(a) * mag).to(x.dtype)[:, None, :]
    half = dims // 2
    if interleaved:
        iu, iv = torch.arange(0, dims, 2), torch.arange(1, dims, 2)
    else:
        iu, iv = torch.arange(0, half), torch.arange(half, dims)
    out = x.clone()
    u, v = x[:, :, iu], x[:, :, iv]
    out[:, :, iu] = u * c - v * s
    out[:, :, iv] = v * c + u * s
    return out


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [S, C], w [C, taps]: y[t] = sum_j w[:, j] u[t - (taps - 1) + j], zeros before the start."""
    S, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < S:
            y[back:] += w[:, j] * u[:S - back]
    return y


def decayed_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [S, H, d], v [S, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    S, H, d = q.shape
    state = torch.zeros((H, d, v.shape[2]), dtype=q.dtype)
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = []
    for t in range(S):
        state = g * state + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", state, q[t]))
    return torch.stack(out)


def gated_recurrence(q: torch.Tensor, f: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q, f [S, H, d], v [S, H, dv]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t."""
    S, H, d = q.shape
    state = torch.zeros((H, d, v.shape[2]), dtype=q.dtype)
    out = []
    for t in range(S):
        state = f[t][:, :, None] * state + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", state, q[t]))
    return torch.stack(out)


def window_visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def mixed_head_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: Optional[float],
                         size: Optional[int], keep_first: int, sink: torch.Tensor, talk: torch.Tensor) -> torch.Tensor:
    """q [S, H, d], k [S, G, d], v [S, G, dv] -> [S, H, dv].  Head h scores against key head h // (H/G); scores are
    scaled, then capped to softcap * tanh(score / softcap); invisible keys drop out; the softmax denominator of head h
    also holds exp(sink[h]); after that the weights of the heads are mixed, w'_h = sum_g talk[h, g] w_g, and head h
    applies w'_h to the values of ITS key/value head.  ``softcap`` None: no cap; ``size`` None: no window."""
    S, H, d = q.shape
    G = k.shape[1]
    per = H // G
    kk = k.repeat_interleave(per, dim=1)                           # [S, H, d]
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap is not None:
        s = softcap * torch.tanh(s / softcap)
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    vis = j <= i
    if size is not None:
        vis = vis & ((i - j < size) | (j < keep_first))
    s = s.masked_fill(~vis[None], float("-inf"))
    m = torch.maximum(s.max(-1).values, sink[:, None])             # [H, S]
    e = torch.exp(s - m[:, :, None])
    w = e / (e.sum(-1) + torch.exp(sink[:, None] - m))[:, :, None]
    w = torch.einsum("hg,gij->hij", talk, w)
    vv = v.repeat_interleave(per, dim=1)                           # [S, H, dv]
    return torch.einsum("hij,jhv->ihv", w, vv)


def two_branch_act(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = F.softplus(p) * z * z + 0.5 * z
    neg = (0.5 + F.softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


# ---------------------------------------------------------------------------
# mixers, feed-forward, model
# ---------------------------------------------------------------------------

def _lin(W: Dict[str, torch.Tensor], name: str, h: torch.Tensor, dt, bias: bool = False) -> torch.Tensor:
    y = h @ W[name].to(dt).t()
    if bias:
        y = y + W[name + ".b"].to(dt)
    return y


def retention_mixer(W, p: str, m: dict, h: torch.Tensor, eps: float, dt=torch.float64) -> torch.Tensor:
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = _lin(W, f"{p}.q", h, dt).view(S, H, d)
    k = _lin(W, f"{p}.k", h, dt).view(S, H, d)
    v = _lin(W, f"{p}.v", h, dt).view(S, H, dv)
    rot = m.get("rot")
    if rot:
        fr, mag = rot_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        pos = torch.arange(S)
        q = rotate(q, pos, rot["dims"], fr, mag, interleaved=False)
        k = rotate(k, pos, rot["dims"], fr, mag, interleaved=False)
    k = k * d ** -0.5
    o = unit_rms(decayed_recurrence(q, k, v, m["decay"]), eps).reshape(S, H * dv)
    return (o * F.silu(_lin(W, f"{p}.g", h, dt))) @ W[f"{p}.o"].to(dt).t()


def left_branch(W, p: str, m: dict, h: torch.Tensor, dt=torch.float64) -> torch.Tensor:
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (_lin(W, f"{p}.{n}", h, dt, bias=True) for n in "qkv")
    if m.get("conv", 1) > 1 or f"{p}.q.conv" in W:
        q, k, v = (short_conv(u, W[f"{p}.{n}.conv"].to(dt)) for n, u in (("q", q), ("k", k), ("v", v)))
    q, k, v = q.view(S, H, d), k.view(S, G, d), v.view(S, G, dv)
    rot = m.get("rot")
    if rot:
        fr, mag = rot_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        pos = torch.arange(S)
        q = rotate(q, pos, rot["dims"], fr, mag, interleaved=True)
        k = rotate(k, pos, rot["dims"], fr, mag, interleaved=True)
    mask = m.get("mask") or {}
    a = mixed_head_attention(q, k, v, m["scale"], m.get("softcap"), mask.get("size"), mask.get("keep_first", 0),
                             W[f"{p}.sink"].to(dt), W[f"{p}.talk"].to(dt))
    return a.reshape(S, H * dv) @ W[f"{p}.o"].to(dt).t()


def right_branch(W, p: str, m: dict, h: torch.Tensor, eps: float, dt=torch.float64) -> torch.Tensor:
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = F.silu(_lin(W, f"{p}.q", h, dt)).view(S, H, d)
    v = _lin(W, f"{p}.v", h, dt).view(S, H, dv)
    low = W[f"{p}.lower"].to(dt)
    f = (low + (1.0 - low) * torch.sigmoid(_lin(W, f"{p}.f", h, dt, bias=True))).view(S, H, d)
    o = unit_rms(gated_recurrence(q, f, v), eps) * W[f"{p}.norm"].to(dt)
    return o.reshape(S, H * dv) @ W[f"{p}.o"].to(dt).t()


def parallel_mixer(W, p: str, m: dict, h: torch.Tensor, eps: float, dt=torch.float64) -> torch.Tensor:
    return (m.get("left_scale", 1.0) * left_branch(W, f"{p}.left", m["left"], h, dt)
            + m.get("right_scale", 1.0) * right_branch(W, f"{p}.right", m["right"], h, eps, dt))


def dense_ff(W, p: str, h: torch.Tensor, dt=torch.float64) -> torch.Tensor:
    act = W[f"{p}.act"].to(dt)
    return two_branch_act(_lin(W, f"{p}.up", h, dt), act[0], act[1]) @ W[f"{p}.down"].to(dt).t()


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, dt=torch.float64, trace: Optional[list] = None) -> torch.Tensor:
    """Logits [S, vocab] of one sequence.  ``trace``: a list that receives the stream [S, width] after every layer."""
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"].to(dt)[tok]

    def norm(name, x):
        return dyn_tanh(x, W[name].to(dt), W[name + ".b"].to(dt), W[name + ".alpha"].to(dt))
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = norm(f"{p}.norm1", x)
        if L["type"] == "retention":
            x = x + retention_mixer(W, f"{p}.mix", L["mixer"], h, eps, dt)
        elif L["type"] == "parallel":
            x = x + parallel_mixer(W, f"{p}.mix", L["mixer"], h, eps, dt)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            x = x + dense_ff(W, f"{p}.mlp", norm(f"{p}.norm2", x), dt)
        if trace is not None:
            trace.append(x.clone())
    return (norm("final.norm", x) @ W["embed"].to(dt).t()) * cfg.get("logit_scale", 1.0)
