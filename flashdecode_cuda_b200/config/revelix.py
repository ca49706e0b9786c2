"""Typed configuration of the Revelix decoder, read from ``config.json``.

The file names the design under ``"architecture"`` and gives every size and
constant per layer: ``layers[i]`` holds ``type`` (which mixer: ``retention`` or
``parallel``), ``mixer`` (its sizes and constants) and ``mlp`` (the
feed-forward, or null); ``norm.eps``, ``vocab``, ``width`` and ``logit_scale``
are global.  A key the design needs and the file lacks is an error that names
its place.  What a file may leave out, with what that means: a mixer's ``rot``
(nothing is rotated), ``rot.scaling`` (plain frequencies), ``mask`` (every
earlier key is visible), ``mask.keep_first`` (none kept), ``softcap`` (scores
are not capped), ``conv`` (one tap: no convolution), the branch scales and
``logit_scale`` (1).  A key this reader does not know changes nothing it
computes; it is kept in ``unknown_keys`` and named in one warning.
"""

from __future__ import annotations

import copy
import warnings
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .qwen2 import ConfigError


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} misses {key!r}")
    return d[key]


_UNKNOWN: List[str] = []       # filled while a configuration is read


def _only(d: Dict[str, Any], known, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    _UNKNOWN.extend(f"{where}.{k}" for k in sorted(set(d) - set(known)))


@dataclass
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Dict[str, float]] = None       # {factor, original, fast, slow} or None

    @classmethod
    def from_dict(cls, r: Optional[Dict[str, Any]], dim: int, where: str) -> Optional["RotationConfig"]:
        if r is None:
            return None
        _only(r, ("dims", "base", "scaling"), where)
        sc = r.get("scaling")
        if sc is not None:
            _only(sc, ("factor", "original", "fast", "slow"), f"{where}.scaling")
            sc = {k: float(_need(sc, k, f"{where}.scaling")) for k in ("factor", "original", "fast", "slow")}
            if not (sc["factor"] > 0 and sc["original"] > 0 and sc["fast"] > 0 and sc["slow"] > 0):
                raise ConfigError(f"config.json: {where}.scaling: every number must be positive")
        c = cls(int(_need(r, "dims", where)), float(_need(r, "base", where)), sc)
        if c.dims <= 0 or c.dims % 2 or c.dims > dim or not c.base > 0 or c.base == 1.0:
            raise ConfigError(f"config.json: {where}: dims must be even, positive and at most dim, base positive and not 1")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(self.scaling)
        return d

    def key(self) -> str:
        sc = "" if self.scaling is None else "@" + ",".join(f"{k}={self.scaling[k]!r}" for k in sorted(self.scaling))
        return f"rot{self.dims}@{self.base!r}{sc}"


@dataclass
class RetentionConfig:
    """Linear attention with a constant decay per head (``layers[i].mixer`` of type ``retention``)."""
    heads: int
    dim: int
    vdim: int
    decay: List[float]
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "RetentionConfig":
        _only(m, ("heads", "dim", "vdim", "decay", "rot"), where)
        dim = int(_need(m, "dim", where))
        c = cls(heads=int(_need(m, "heads", where)), dim=dim, vdim=int(_need(m, "vdim", where)),
                decay=[float(g) for g in _need(m, "decay", where)],
                rot=RotationConfig.from_dict(m.get("rot"), dim, f"{where}.rot"))
        if min(c.heads, c.dim, c.vdim) <= 0 or len(c.decay) != c.heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and 'decay' hold one number per head")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class SinkAttentionConfig:
    """The attention branch of a ``parallel`` mixer (``mixer.left``)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    keep_first: int
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "SinkAttentionConfig":
        _only(m, ("heads", "kv_heads", "dim", "vdim", "conv", "rot", "scale", "softcap", "mask"), where)
        mask = m.get("mask")
        if mask is not None:
            _only(mask, ("size", "keep_first"), f"{where}.mask")
        dim = int(_need(m, "dim", where))
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=dim,
                vdim=int(_need(m, "vdim", where)), conv=int(m.get("conv", 1)), scale=float(_need(m, "scale", where)),
                softcap=None if m.get("softcap") is None else float(m["softcap"]),
                window=None if mask is None else int(_need(mask, "size", f"{where}.mask")),
                keep_first=0 if mask is None else int(mask.get("keep_first", 0)),
                rot=RotationConfig.from_dict(m.get("rot"), dim, f"{where}.rot"))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv, 1 if c.window is None else c.window) <= 0 \
                or c.heads % c.kv_heads or c.keep_first < 0 or (c.softcap is not None and not c.softcap > 0):
            raise ConfigError(f"config.json: {where}: sizes and the soft cap must be positive, heads a multiple of "
                              f"kv_heads, keep_first not negative")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                             "scale": self.scale, "vdim": self.vdim}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window is not None:
            d["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class GatedRecurrenceConfig:
    """The recurrent branch of a ``parallel`` mixer (``mixer.right``)."""
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "GatedRecurrenceConfig":
        _only(m, ("heads", "dim", "vdim"), where)
        c = cls(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "vdim", where)))
        if min(c.heads, c.dim, c.vdim) <= 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass
class ParallelConfig:
    """Two mixers on the same input, their outputs added with fixed weights (type ``parallel``)."""
    left: SinkAttentionConfig
    right: GatedRecurrenceConfig
    left_scale: float = 1.0
    right_scale: float = 1.0

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "ParallelConfig":
        _only(m, ("left", "right", "left_scale", "right_scale"), where)
        return cls(SinkAttentionConfig.from_dict(_need(m, "left", where), f"{where}.left"),
                   GatedRecurrenceConfig.from_dict(_need(m, "right", where), f"{where}.right"),
                   float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass
class DenseFFConfig:
    ff: int

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "DenseFFConfig":
        _only(m, ("kind", "ff"), where)
        if _need(m, "kind", where) != "dense":
            raise ConfigError(f"config.json: {where}.kind {m['kind']!r}: this design's feed-forward is 'dense'")
        c = cls(int(_need(m, "ff", where)))
        if c.ff <= 0:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


@dataclass
class RevelixLayer:
    type: str
    mixer: Any                          # RetentionConfig or ParallelConfig
    mlp: Optional[DenseFFConfig]


@dataclass
class RevelixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[RevelixLayer]
    logit_scale: float = 1.0
    eos_token_id: Optional[Any] = None
    architecture: str = "Revelix"
    unknown_keys: List[str] = field(default_factory=list)

    MIXERS = {"retention": RetentionConfig, "parallel": ParallelConfig}

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "RevelixConfig":
        _UNKNOWN.clear()
        _only(cfg, ("architecture", "architectures", "layers", "norm", "vocab", "width", "logit_scale", "eos_token_id"),
              "the top level")
        raw_layers = _need(cfg, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(L, ("type", "mixer", "mlp"), where)
            kind = _need(L, "type", where)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r}: this design's mixers are {sorted(cls.MIXERS)}")
            mixer = cls.MIXERS[kind].from_dict(_need(L, "mixer", where), f"{where}.mixer")
            mlp = L.get("mlp")
            layers.append(RevelixLayer(kind, mixer, None if mlp is None else DenseFFConfig.from_dict(mlp, f"{where}.mlp")))
        out = cls(vocab=int(_need(cfg, "vocab", "the top level")), width=int(_need(cfg, "width", "the top level")),
                  norm_eps=float(_need(_need(cfg, "norm", "the top level"), "eps", "norm")), layers=layers,
                  logit_scale=float(cfg.get("logit_scale", 1.0)), eos_token_id=cfg.get("eos_token_id"))
        if out.vocab <= 0 or out.width <= 0 or not out.norm_eps > 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        out.unknown_keys = list(_UNKNOWN)
        if out.unknown_keys:
            warnings.warn(f"config.json has keys the Revelix design does not define (ignored): {out.unknown_keys}")
        return out

    def stop_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers],
            "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
        }
        if self.eos_token_id is not None:
            d["eos_token_id"] = copy.deepcopy(self.eos_token_id)
        return d

    def summary(self) -> str:
        kinds = ", ".join(f"{sum(L.type == k for L in self.layers)} {k}" for k in sorted(self.MIXERS))
        return (f"Revelix layers={len(self.layers)} ({kinds}) width={self.width} vocab={self.vocab} "
                f"eps={self.norm_eps} logit_scale={self.logit_scale}")
