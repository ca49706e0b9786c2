"""Shared by the Revelix tests: small configurations that differ from one another in every size and option, model
folders with random weights, the plain implementation as ground truth."""

from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Optional

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint
from plain import revelix_plain as P


def _rot(dims, base, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def retention(heads, dim, vdim, decay, rot=None, mlp=None):
    m = {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}
    if rot is not None:
        m["rot"] = rot
    return {"type": "retention", "mixer": m, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, conv, scale, softcap=None, window=None, keep_first=None, rot=None):
    m = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot is not None:
        m["rot"] = rot
    return m


def recurrence(heads, dim, vdim):
    return {"dim": dim, "heads": heads, "vdim": vdim}


def parallel(left, right, left_scale=None, right_scale=None, mlp=None):
    m = {"left": left, "right": right}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return {"type": "parallel", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def model(vocab, width, eps, layers, logit_scale=None):
    cfg = {"architecture": "Revelix", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


REVELIX: Dict[str, dict] = {
    # a parallel layer first and a retention layer last; value heads wider than key heads on the left and narrower on
    # the right; three query heads per key head; four taps; half of each head rotated with stretched frequencies; a
    # window that is no multiple of a page with a few kept positions; retention with a feed-forward and a partial rotation
    "P": model(211, 96, 1e-6, [
        parallel(attention(6, 2, 32, 40, 4, 0.2, softcap=8.0, window=27, keep_first=5,
                           rot=_rot(16, 10000.0, (4.0, 64, 16.0, 2.0))),
                 recurrence(3, 24, 16), 0.7, 1.3, mlp=dense(136)),
        retention(4, 24, 40, [0.9, 0.97, 0.99, 0.999], rot=_rot(8, 500.0), mlp=dense(72)),
    ], logit_scale=0.5),
    # one key head for all query heads; one tap (no convolution state); nothing rotated on the left; a window of one
    # page exactly and nothing kept; no soft cap; the branch scales and the logit scale left to their default of one;
    # retention without rotation, with one head; a parallel layer without a feed-forward
    "Q": model(96, 64, 1e-5, [
        retention(1, 64, 64, [0.95]),
        parallel(attention(4, 1, 64, 64, 1, 0.125, window=16, keep_first=0), recurrence(1, 64, 64)),
        parallel(attention(4, 1, 64, 64, 1, 0.125, window=16, keep_first=0), recurrence(1, 64, 64), mlp=dense(64)),
    ]),
    # one query head per key head; two taps; every dimension rotated, plain frequencies; kept positions beyond the
    # window's size; head sizes that are multiples of 8 only; a width that is no multiple of 16; no window at all on
    # the last layer's attention; retention heads wider than 128
    "R": model(160, 72, 1e-5, [
        retention(2, 136, 24, [0.5, 1.0], rot=_rot(136, 1000000.0)),
        parallel(attention(3, 3, 24, 8, 2, 0.3, softcap=30.0, window=9, keep_first=14, rot=_rot(24, 100.0)),
                 recurrence(2, 8, 48), 1.5, 0.25, mlp=dense(40)),
        parallel(attention(2, 2, 40, 24, 5, 0.11, softcap=2.0, rot=_rot(2, 10000.0, (16.0, 32, 4.0, 1.0))),
                 recurrence(4, 40, 8), 1.0, 1.0, mlp=None),
    ], logit_scale=3.0),
}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: layer orders of every kind, widths that are no power of two, head counts
    and sizes of all three mixers drawn apart, one to five taps, nothing to everything rotated with and without
    stretched frequencies, windows from one position to longer than any test sequence, kept positions from none to
    more than the window, layers with and without a feed-forward."""
    rng = random.Random(seed)
    width = rng.choice([48, 72, 96, 128, 200, 256])

    def rot(dim, may_scale=True):
        if rng.random() < 0.15:
            return None
        dims = min(dim, rng.choice([2, 4, 8, 16, dim]))
        dims -= dims % 2
        sc = None
        if may_scale and rng.random() < 0.6:
            sc = (rng.choice([2.0, 8.0, 32.0]), rng.choice([16, 64, 1024]), rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0]))
        return _rot(dims, rng.choice([100.0, 10000.0, 1000000.0]), sc)

    def mlp():
        return None if rng.random() < 0.3 else dense(rng.choice([8, 24, 40, 96, 100, 264]))

    def ret():
        h, d = rng.choice([1, 2, 3, 5]), rng.choice([8, 12, 16, 24, 40, 64, 128, 136])
        return retention(h, d, rng.choice([6, 8, 16, 24, 64, 72]), [rng.choice([0.5, 0.9, 0.99, 0.9995, 1.0]) for _ in range(h)],
                         rot(d, may_scale=False), mlp())

    def par():
        kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
        d = rng.choice([8, 12, 16, 20, 24, 32, 40, 64, 128])
        window = rng.choice([None, 1, 2, 7, 16, 33, 64, 100, 1000])
        keep = None if window is None else rng.choice([None, 0, 1, 4, 17, 40])
        left = attention(kv * g, kv, d, rng.choice([d, 8, 12, 16, 48, 64]), rng.choice([1, 2, 3, 4, 5]),
                         rng.choice([0.1, 0.125, 0.3]), rng.choice([None, 1.0, 5.0, 50.0]), window, keep, rot(d))
        right = recurrence(rng.choice([1, 2, 3]), rng.choice([8, 10, 16, 24, 48, 64, 136]), rng.choice([4, 8, 16, 32, 40, 64]))
        return parallel(left, right, rng.choice([None, 0.5, 1.0, 2.0]), rng.choice([None, 0.3, 1.0, 1.7]), mlp())
    layers = [ret() if rng.random() < 0.45 else par() for _ in range(rng.randint(1, 4))]
    return model(rng.choice([50, 333, 1000]), width, rng.choice([1e-5, 1e-6]), layers, rng.choice([None, 0.25, 1.0, 4.0]))


def write_folder(tmp: Path, name: str, seed: int = 0) -> Path:
    folder = Path(tmp) / f"revelix_{name}_{seed}"
    if not (folder / "model.safetensors").exists():
        fd.write_random_model(folder, REVELIX[name], seed)
    return folder


def raw_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def weights_of(folder: Path) -> Dict[str, torch.Tensor]:
    return {k: v.clone() for k, v in load_checkpoint(folder).items()}


_ORACLE: dict = {}

# The plain model in float32 lies this far (relative to the largest logit) from the plain model in float64 where nothing
# amplifies rounding; the configurations of this file measure 2e-7 to 9e-7.
SINGLE_PRECISION_DISTANCE = 5e-7
# Whole models, relative to the largest logit of the sequence, where nothing amplifies rounding.  float32: only the
# order of summation differs from the float64 ground truth.  bfloat16: products and activations are rounded to 8 bits of
# mantissa layer after layer; what a wrong mask, state or page does is told apart by the float32 runs and by the kernel
# tests with keys that stand out.
MODEL_TOL = {"float32": 1e-4, "bfloat16": 5e-2}


class Truth:
    """The float64 logits [len, vocab] of one whole sequence from the plain implementation, and for every position how
    far rounding alone moves it: the distance of the plain model run in float32.  With random weights a position now
    and then divides by a root mean square of terms that nearly cancel (a head's output before its unit norm), and
    every rounding before it is magnified there, in any implementation; such a position is allowed that much more."""

    def __init__(self, cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int]):
        self.logits = P.forward(cfg, W, tokens)
        self.scale = max(float(self.logits.abs().max()), 1e-6)
        single = P.forward(cfg, W, tokens, dt=torch.float32).double()
        self.single = (single - self.logits).abs().amax(-1) / self.scale               # [len]

    def allowed(self, dtype: str) -> torch.Tensor:
        """[len]: the largest relative distance a position may have in ``dtype``."""
        if dtype == "float32":
            return torch.clamp(6 * self.single, min=MODEL_TOL[dtype])
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
    """float64 logits [len, vocab] of one whole sequence from the plain implementation."""
    return truth(folder, tokens).logits


def plain_greedy(folder: Path, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(oracle_logits(folder, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
