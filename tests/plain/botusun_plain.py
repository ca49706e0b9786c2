"""Plain, slow implementation of the Botusun decoder: whole sequences, no cache,
one function per mechanism.  It shares no code with the product package; it
reads a raw ``config.json`` dictionary and a ``{tensor name: tensor}`` dict.

Botusun in this file's notation.  The stream starts as embed[token] * s_e.  A
layer is pre-norm with one multiplier m on everything it adds:
x += m * mixer(n1(x)); x += m * ff(n2(x)) where the layer has a feed-forward;
then the token's own contribution, x += m * unit_rms(y) * w_s with
y = P (gelu(G x) * e_l[token]), e_l being the layer's slice of a second
embedding table.  n(x) = x / sqrt(mean(x^2) + eps) * w.  Two kinds of mixer:

* ``gla``: linear attention with a decay per key channel,
  S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, where
  a = sigmoid(A2 (A1 h) + b)^(1/tau) and q is scaled by dim^(-1/2); every head's
  output is RMS-normed with one weight vector, the heads are multiplied by
  silu(W_g h) and projected.
* ``attention``: grouped-head softmax attention whose q and k (biased) pass a
  short causal convolution over time, then an RMS norm per head, then a rotation
  of the leading dimensions (pairs (i, i + dims/2)) whose slow frequencies are
  divided by a factor, fast ones kept and the ones between blended.  The values
  are the convolved keys as they were before norm and rotation.  A query sees
  itself and the window's other positions before it; the softmax denominator
  has one more term, 1.

The feed-forward is gated, down(silu(gate h) * (up h)), dense or as a mixture
of experts: sigmoid router scores, a choice by score + correction restricted to
the best groups of neighbouring experts (a group's rank is the sum of its two
largest choice scores), weights = the plain scores of the chosen, times a
constant.  A span of layers may run several times with the same weights; every
pass starts by adding a vector of its own to the stream.  The logits are the
final norm's output times the embedding table (unscaled).

The arithmetic dtype is a parameter (float64 by default).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rot_frequencies(dims: int, base: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2.  With ``scaling`` (factor, low, high, original), by the wavelength
    l = 2 pi / f: l < original / high keeps f; l > original / low gives f / factor; between them
    s = (original / l - low) / (high - low) blends (1 - s) f / factor + s f."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, lo, hi = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            orig = float(scaling["original"])
            wl = 2.0 * math.pi / f
            if wl < orig / hi:
                pass
            elif wl > orig / lo:
                f = f / factor
            else:
                s = (orig / wl - lo) / (hi - lo)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, freqs: torch.Tensor) -> torch.Tensor:
    """x [S, heads, d]: dimension i < dims/2 of each head is paired with i + dims/2;
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i.  Dimensions from ``dims`` on pass."""
    if not dims:
        return x
    a = positions.to(torch.float64)[:, None] * freqs[None, :]
    c, s = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    half = dims // 2
    out = x.clone()
    u, v = x[:, :, :half], x[:, :, half:dims]
    out[:, :, :half] = u * c - v * s
    out[:, :, half:dims] = v * c + u * s
    return out


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [S, C], w [C, taps]: y[t] = sum_j w[:, j] u[t - (taps - 1) + j], zeros before the start."""
    S = u.shape[0]
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < S:
            y[back:] += w[:, j] * u[:S - back]
    return y


def channel_decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                             state: Optional[torch.Tensor] = None):
    """q, k, a [S, H, d], v [S, H, dv]: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token.
    Returns (o [S, H, dv], the last state)."""
    S, H, d = q.shape
    if state is None:
        state = torch.zeros((H, d, v.shape[2]), dtype=q.dtype)
    out = []
    for t in range(S):
        state = a[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", state, q[t]))
    return torch.stack(out), state


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                           window: Optional[int]) -> torch.Tensor:
    """q [S, H, d], k [S, G, d], v [S, G, dv]; query head h reads key/value head h // (H / G).  The query at i
    sees j with 0 <= i - j < window (every j <= i without one).  p_j = exp(s_j) / (1 + sum_j exp(s_j))."""
    S, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(S):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = torch.clamp(s.max(), min=0.0)                  # the keyless term has score 0
            e = torch.exp(s - m)
            p = e / (torch.exp(-m) + e.sum())
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def gla_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mc: dict, eps: float,
              capture: Optional[dict] = None) -> torch.Tensor:
    S = h.shape[0]
    H, d, dv, tau = mc["heads"], mc["dim"], mc["vdim"], float(mc["tau"])
    q = (h @ W[f"{p}.q"].T).view(S, H, d) * d ** -0.5
    k = (h @ W[f"{p}.k"].T).view(S, H, d)
    v = (h @ W[f"{p}.v"].T).view(S, H, dv)
    z = (h @ W[f"{p}.a1"].T) @ W[f"{p}.a2"].T + W[f"{p}.a2.b"]
    a = torch.sigmoid(z).pow(1.0 / tau).view(S, H, d)
    o, _ = channel_decay_recurrence(q, k, v, a)
    if capture is not None:
        capture.update(q=q, k=k, v=v, a=a, o=o)
    o = rms_norm(o, W[f"{p}.norm"], eps).reshape(S, H * dv)
    return (o * silu(h @ W[f"{p}.g"].T)) @ W[f"{p}.o"].T


def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mc: dict, eps: float,
                    capture: Optional[dict] = None) -> torch.Tensor:
    S = h.shape[0]
    H, G, d = mc["heads"], mc.get("kv_heads", mc["heads"]), mc["dim"]
    q = h @ W[f"{p}.q"].T + W[f"{p}.q.b"]
    k = h @ W[f"{p}.k"].T + W[f"{p}.k.b"]
    q = short_conv(q, W[f"{p}.q.conv"]).view(S, H, d)
    k = short_conv(k, W[f"{p}.k.conv"]).view(S, G, d)
    v = k                                                       # the values: the convolved keys, nothing more
    qn, kn = rms_norm(q, W[f"{p}.q.norm"], eps), rms_norm(k, W[f"{p}.k.norm"], eps)
    rot = mc.get("rot")
    if rot:
        f = rot_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        pos = torch.arange(S)
        qn, kn = rotate_half(qn, pos, rot["dims"], f), rotate_half(kn, pos, rot["dims"], f)
    window = mc["mask"]["size"] if mc.get("mask") else None
    o = sink_softmax_attention(qn, kn, v, float(mc["scale"]), window)
    if capture is not None:
        capture.update(q=qn, k=kn, v=v, o=o)
    return o.reshape(S, -1) @ W[f"{p}.o"].T


def gated_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, rc: dict):
    """(chosen expert ids [S, top], their weights [S, top]) for the rows of h."""
    E, top = rc["experts"], rc["top"]
    s = torch.sigmoid(h @ router.T)                              # [S, E]
    choice = s + correction
    groups = rc.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        grouped = choice.view(-1, n, per)
        rank = grouped.topk(min(2, per), dim=-1).values.sum(-1)                  # [S, n]
        best = rank.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(rank, dtype=torch.bool).scatter_(1, best, True)
        choice = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), choice,
                             torch.full_like(choice, -math.inf))
    ids = choice.topk(top, dim=-1).indices
    return ids, s.gather(1, ids) * float(rc.get("scale", 1.0))


def moe_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, fc: dict, capture: Optional[dict] = None):
    rc = fc["router"]
    ids, w = route(h, W[f"{p}.router"], W[f"{p}.correction"], rc)
    if capture is not None:
        capture.update(ids=ids, weights=w)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            q = f"{p}.e{e}"
            out[t] += we * gated_ff(h[t:t + 1], W[f"{q}.gate"], W[f"{q}.up"], W[f"{q}.down"])[0]
    return out


def token_side(x: torch.Tensor, tokens: torch.Tensor, W: Dict[str, torch.Tensor], layer: int, dim: int,
               eps: float) -> torch.Tensor:
    """What a layer adds (before the multiplier) from the token itself: unit_rms(P (gelu(G x) * e)) * w."""
    p = f"l{layer}.side"
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[f"{p}.gate"].T) * e) @ W[f"{p}.proj"].T
    return rms_norm(y, W[f"{p}.norm"], eps)


def layer_runs(cfg: dict) -> List[tuple]:
    """[(layer, pass number or None)]: the order in which layers run; the pass number is set on the first layer
    of every pass of the looped span."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False,
            captures: Optional[list] = None):
    """Logits [S, vocab] of one whole sequence (and, on request, the stream after every layer run).  ``captures``: a
    list that receives (layer, type, what the mixer saw) for every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = W["embed"][tokens] * float(cfg.get("embedding", {}).get("scale", 1.0))
    side = cfg.get("token_side")
    layers = []
    for i, t in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}"
        if t is not None:
            x = x + W["loop.step"][t]
        h = rms_norm(x, W[f"{p}.norm1"], eps)
        cap = None if captures is None else {}
        if L["type"] == "gla":
            x = x + m * gla_mixer(h, W, f"{p}.mix", L["mixer"], eps, cap)
        elif L["type"] == "attention":
            x = x + m * attention_mixer(h, W, f"{p}.mix", L["mixer"], eps, cap)
        else:
            raise ValueError(L["type"])
        if captures is not None:
            captures.append((i, L["type"], cap))
        fc = L.get("mlp")
        if fc:
            h = rms_norm(x, W[f"{p}.norm2"], eps)
            if fc["kind"] == "dense":
                x = x + m * gated_ff(h, W[f"{p}.mlp.gate"], W[f"{p}.mlp.up"], W[f"{p}.mlp.down"])
            else:
                x = x + m * moe_ff(h, W, f"{p}.mlp", fc)
        if side:
            x = x + m * token_side(x, tokens, W, i, side["dim"], eps)
        layers.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, torch.stack(layers)) if return_layers else logits
