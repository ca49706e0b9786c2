"""Shared by the Botusun tests: small configurations that differ from one another in every size and option, model
folders with random weights, the plain implementation as ground truth."""

from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Optional

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint, write_model_folder
from plain import botusun_plain as P


def rot(dims, base, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def gla(heads, dim, vdim, tau, rank, mlp=None):
    return {"type": "gla", "mixer": {"dim": dim, "heads": heads, "rank": rank, "tau": tau, "vdim": vdim}, "mlp": mlp}


def attention(heads, kv_heads, dim, conv, scale, window=None, rotation=None, mlp=None):
    m = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": dim}
    if window is not None:
        m["mask"] = {"size": window}
    if rotation is not None:
        m["rot"] = rotation
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, groups=None, scale=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    return {"expert": {"ff": ff}, "kind": "moe", "router": r}


def model(vocab, width, eps, layers, mult=None, emb_scale=None, side=None, loop=None):
    cfg = {"architecture": "Botusun", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if mult is not None:
        cfg["residual_mult"] = mult
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


BOTUSUN: Dict[str, dict] = {
    # attention first, a loop of two passes over the last two layers (an attention and a linear-attention layer, each pass
    # with its own pages and states), three query heads per key head, three taps, a quarter of each head rotated with
    # scaled frequencies, a window that is no multiple of a page, six experts in three groups of which two are kept,
    # value heads of the linear attention wider than its key heads, a side table of 8 columns per layer
    "A": model(211, 96, 1e-6, [
        attention(6, 2, 32, 3, 0.2, window=27, rotation=rot(8, 10000.0, (8.0, 1.0, 4.0, 64)), mlp=dense(136)),
        attention(2, 1, 24, 2, 0.3, window=40, rotation=rot(24, 500.0), mlp=moe(6, 2, 40, groups=(3, 2), scale=1.5)),
        gla(3, 24, 40, 8.0, 12, mlp=moe(6, 3, 24, groups=(2, 1), scale=0.5)),
    ], mult=0.5, emb_scale=3.0, side=8, loop=(1, 3, 2)),
    # no loop, no side input, multiplier and embedding scale left at one; one key head for all query heads, one tap (no
    # convolution state), nothing rotated, a window of one page exactly; a layer without a feed-forward; groups of one
    # expert each (a group's rank is its one score); one choice per token; no groups at all
    "B": model(96, 64, 1e-5, [
        gla(1, 64, 64, 1.0, 4),
        attention(4, 1, 64, 1, 0.125, window=16, mlp=moe(4, 1, 16, groups=(4, 2))),
        gla(2, 16, 8, 30.0, 32, mlp=moe(5, 2, 8)),
        attention(4, 4, 16, 4, 0.25, mlp=dense(64)),
    ]),
    # the whole model is the loop, three passes; head sizes that are multiples of 8 only and a width that is no multiple
    # of 16; every dimension rotated; no window at all; a window of one position (a query sees itself alone); five taps;
    # key heads of the linear attention wider than 128
    "C": model(160, 72, 1e-5, [
        gla(2, 136, 24, 4.0, 8, mlp=dense(40)),
        attention(3, 3, 24, 5, 0.3, rotation=rot(24, 100.0, (2.0, 2.0, 8.0, 16)), mlp=None),
        attention(2, 2, 40, 2, 0.11, window=1, rotation=rot(2, 10000.0), mlp=moe(8, 4, 16, groups=(4, 3), scale=2.5)),
    ], mult=0.25, emb_scale=7.0, side=5, loop=(0, 3, 3)),
}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: layer orders of every kind, widths that are no power of two, head counts and
    sizes of both mixers drawn apart, one to five taps, nothing to everything rotated with and without scaled
    frequencies, windows from one position to longer than any test sequence, dense and routed feed-forwards and none,
    loops over any span (also all layers, also once), with and without the side input."""
    rng = random.Random(seed)
    width = rng.choice([36, 48, 72, 96, 100, 128, 200, 256])

    def rotation(dim):
        if rng.random() < 0.15:
            return None
        dims = min(dim, rng.choice([2, 4, 8, 16, dim]))
        dims -= dims % 2
        sc = None
        if rng.random() < 0.6:
            low = rng.choice([0.5, 1.0, 2.0])
            sc = (rng.choice([2.0, 8.0, 32.0]), low, low * rng.choice([2.0, 4.0, 8.0]), rng.choice([16, 64, 1024]))
        return rot(dims, rng.choice([100.0, 10000.0, 1000000.0]), sc)

    def mlp():
        x = rng.random()
        if x < 0.2:
            return None
        if x < 0.5:
            return dense(rng.choice([8, 24, 40, 96, 100, 264]))
        groups = rng.choice([None, 1, 2, 3, 4])
        per = rng.choice([1, 2, 3, 4])
        experts = per * (groups or rng.choice([1, 2, 5]))
        keep = None if groups is None else rng.randint(1, groups)
        top = rng.randint(1, min(4, per * (keep or 1) if groups else experts))
        return moe(experts, top, rng.choice([8, 12, 16, 40, 64]), None if groups is None else (groups, keep),
                   rng.choice([None, 0.5, 1.0, 2.5]))

    def lin():
        return gla(rng.choice([1, 2, 3, 5]), rng.choice([8, 12, 16, 24, 40, 64, 128, 136]), rng.choice([6, 8, 16, 24, 64, 72]),
                   rng.choice([1.0, 4.0, 16.0, 64.0]), rng.choice([1, 4, 16, 24]), mlp())

    def att():
        kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
        d = rng.choice([8, 12, 16, 20, 24, 32, 40, 64, 128])
        return attention(kv * g, kv, d, rng.choice([1, 2, 3, 4, 5]), rng.choice([0.1, 0.125, 0.3]),
                         rng.choice([None, 1, 2, 7, 16, 33, 64, 100, 1000]), rotation(d), mlp())
    n = rng.randint(1, 4)
    layers = [lin() if rng.random() < 0.45 else att() for _ in range(n)]
    loop = None
    if rng.random() < 0.7:
        start = rng.randint(0, n - 1)
        loop = (start, rng.randint(start + 1, n), rng.randint(1, 3))
    return model(rng.choice([50, 333, 1000]), width, rng.choice([1e-5, 1e-6]), layers, rng.choice([None, 0.3, 1.0, 0.7]),
                 rng.choice([None, 1.0, 12.0]), rng.choice([None, 1, 4, 16, 20]), loop)


def decisive_corrections(folder: Path) -> Path:
    """Rewrite every router's corrections so that they alone decide the choice: steps of 3 between the experts of a
    group and far larger steps between the groups, while scores lie in (0, 1).  In bfloat16 a choice between two
    nearly equal scores, or between two groups whose ranks nearly tie, falls either way and says nothing about the
    kernels."""
    cfg = raw_config(folder)
    W = weights_of(folder)
    for name in [n for n in W if n.endswith(".correction")]:
        layer = int(name.split(".")[0][1:])
        n = W[name].numel()
        groups = (cfg["layers"][layer]["mlp"]["router"].get("groups") or {"count": 1})["count"]
        per = n // groups
        g = torch.Generator().manual_seed(n + 7 * layer)
        order = torch.randperm(groups, generator=g)
        corr = torch.zeros(n)
        for k in range(groups):
            corr[k * per:(k + 1) * per] = 3.0 * (order[k] * 2 * per + torch.randperm(per, generator=g)).float()
        W[name] = corr.to(W[name].dtype)
    write_model_folder(folder, cfg, W)
    return folder


def write_folder(tmp: Path, name: str, seed: int = 0, decisive: bool = False) -> Path:
    folder = Path(tmp) / f"botusun_{name}_{seed}{'_d' if decisive else ''}"
    if not (folder / "model.safetensors").exists():
        fd.write_random_model(folder, BOTUSUN[name], seed)
        if decisive:
            decisive_corrections(folder)
    return folder


def raw_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def weights_of(folder: Path) -> Dict[str, torch.Tensor]:
    return {k: v.clone() for k, v in load_checkpoint(folder).items()}


_ORACLE: dict = {}

SINGLE_PRECISION_DISTANCE = 5e-7
# |cos| of the angle between the first token's q and k of a linear-attention head below which bfloat16 may flip the
# sign of that head's first output (see ``Truth``); about one sequence in five has such a head among half a dozen
FIRST_TOKEN_MARGIN = 0.01
# Whole models, relative to the largest logit of the sequence, where nothing amplifies rounding.  float32: only the
# order of summation differs from the float64 ground truth.  bfloat16: products and activations are rounded to 8 bits
# of mantissa layer after layer, and this design renormalises vectors that partly cancel in every layer (each q and k
# head after its convolution, the token's own contribution over its root mean square): the library's bfloat16 path
# measures 0.01 to 0.07 on these configurations where the plain model run wholly in bfloat16 lies at 0.05 to 0.5.  What
# a wrong mask, state or page does is told apart by the float32 runs and by the kernel tests with keys that stand out.
MODEL_TOL = {"float32": 1e-4, "bfloat16": 8e-2}


class Truth:
    """The float64 logits [len, vocab] of one whole sequence from the plain implementation, and for every position how
    far rounding alone moves it: the distance of the plain model run in float32.  Where random weights make a norm
    divide by a root mean square of terms that nearly cancel, every rounding before it is magnified, in any
    implementation; such a position is allowed that much more."""

    def __init__(self, cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int]):
        captures: list = []
        self.logits = P.forward(cfg, W, tokens, captures=captures)
        self.scale = max(float(self.logits.abs().max()), 1e-6)
        # The first token's output of a linear-attention head is (q . k) v, and the norm that follows leaves v / rms(v)
        # times the SIGN of q . k: where q and k are nearly at right angles, rounding to 8 bits decides that sign, and
        # the state carries the difference on.  Such a sequence says nothing about the bfloat16 path.
        self.first_margin = 1.0
        for _, kind, cap in captures:
            if kind == "gla":
                q0, k0 = cap["q"][0], cap["k"][0]
                cos = (q0 * k0).sum(-1).abs() / (q0.norm(dim=-1) * k0.norm(dim=-1) + 1e-30)
                self.first_margin = min(self.first_margin, float(cos.min()))
        single = P.forward(cfg, W, tokens, dtype=torch.float32).double()
        self.single = (single - self.logits).abs().amax(-1) / self.scale               # [len]

    def allowed(self, dtype: str) -> torch.Tensor:
        if dtype == "float32":
            return torch.clamp(6 * self.single, min=MODEL_TOL[dtype])
        if self.first_margin < FIRST_TOKEN_MARGIN:
            return torch.full_like(self.single, float("inf"))
        return MODEL_TOL[dtype] * torch.clamp(self.single / SINGLE_PRECISION_DISTANCE, min=1.0)

    def excess(self, got: torch.Tensor, rows, dtype: str) -> float:
        """max over the rows of ``got`` (logits at the positions ``rows``) of distance / allowed distance: below 1
        passes."""
        rows = list(rows)
        got = got.detach().double().cpu().reshape(len(rows), -1)
        d = (got - self.logits[rows]).abs().amax(-1) / self.scale
        return float((d / self.allowed(dtype)[rows]).max())


def truth(folder: Path, tokens: List[int]) -> Truth:
    key = (str(folder), tuple(tokens))
    if key not in _ORACLE:
        _ORACLE[key] = Truth(raw_config(folder), weights_of(folder), tokens)
    return _ORACLE[key]


def oracle_logits(folder: Path, tokens: List[int]) -> torch.Tensor:
    return truth(folder, tokens).logits


def plain_greedy(folder: Path, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(oracle_logits(folder, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
