"""Typed configuration of the Botusun decoder, read from ``config.json``.

The file names the design under ``"architecture"`` and gives every size and
constant: ``layers[i]`` holds ``type`` (which mixer: ``gla`` or ``attention``),
``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, ``kind``
``dense`` or ``moe``, or null); ``loop`` (``start``, ``stop``, ``times``) names
a span of layers that runs several times with the same weights;
``embedding.scale``, ``residual_mult``, ``norm.eps``, ``token_side.dim``,
``vocab`` and ``width`` are global.  A key the design needs and the file lacks
is an error that names its place.  What a file may leave out, with what that
means: ``loop`` (every layer runs once), ``token_side`` (layers add nothing
from the token itself), ``embedding.scale`` and ``residual_mult`` (1), an
attention mixer's ``rot`` (nothing is rotated), ``rot.scaling`` (plain
frequencies), ``mask`` (every earlier key is visible), ``conv`` (one tap: no
convolution), ``kv_heads`` (as many as ``heads``), a ``gla`` mixer's ``rank`` (the rows of its narrow decay
projection: the checkpoint's tensors give them; random weights need the key), a router's ``groups`` (every
expert can be chosen) and ``scale`` (1).  A key this reader does not know
changes nothing it computes; it is kept in ``unknown_keys`` and named in one
warning.
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
class WavelengthRotation:
    """A rotation of the first ``dims`` dimensions of a head whose slow frequencies may be divided by a factor
    (``scaling`` = {factor, low, high, original}, by wavelength)."""
    dims: int
    base: float
    scaling: Optional[Dict[str, float]] = None

    @classmethod
    def from_dict(cls, r: Optional[Dict[str, Any]], dim: int, where: str) -> Optional["WavelengthRotation"]:
        if r is None:
            return None
        _only(r, ("dims", "base", "scaling"), where)
        sc = r.get("scaling")
        if sc is not None:
            _only(sc, ("factor", "low", "high", "original"), f"{where}.scaling")
            sc = {k: float(_need(sc, k, f"{where}.scaling")) for k in ("factor", "low", "high", "original")}
            if not (sc["factor"] > 0 and sc["original"] > 0 and sc["low"] > 0 and sc["high"] > 0):
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
class ChannelDecayConfig:
    """Linear attention with a decay per key channel (``layers[i].mixer`` of type ``gla``)."""
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None      # rows of the decay's narrow projection; None: the checkpoint's tensors give it

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "ChannelDecayConfig":
        _only(m, ("heads", "dim", "vdim", "tau", "rank"), where)
        c = cls(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "vdim", where)),
                float(_need(m, "tau", where)), None if m.get("rank") is None else int(m["rank"]))
        if min(c.heads, c.dim, c.vdim, 1 if c.rank is None else c.rank) <= 0 or not c.tau > 0:
            raise ConfigError(f"config.json: {where}: sizes and tau must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass
class NormedConvAttentionConfig:
    """Windowed softmax attention over convolved, normed, rotated q and k whose values are the convolved keys
    (``layers[i].mixer`` of type ``attention``)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    window: Optional[int]
    rot: Optional[WavelengthRotation]

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "NormedConvAttentionConfig":
        _only(m, ("heads", "kv_heads", "dim", "vdim", "conv", "rot", "scale", "mask"), where)
        mask = m.get("mask")
        if mask is not None:
            _only(mask, ("size",), f"{where}.mask")
        dim, heads = int(_need(m, "dim", where)), int(_need(m, "heads", where))
        c = cls(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=dim, vdim=int(m.get("vdim", dim)),
                conv=int(m.get("conv", 1)), scale=float(_need(m, "scale", where)),
                window=None if mask is None else int(_need(mask, "size", f"{where}.mask")),
                rot=WavelengthRotation.from_dict(m.get("rot"), dim, f"{where}.rot"))
        if min(c.heads, c.kv_heads, c.dim, c.conv, 1 if c.window is None else c.window) <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if c.vdim != c.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim ({c.vdim}) must equal dim ({c.dim})")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                             "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class GatedFFConfig:
    """``mlp`` of kind ``dense``: down(silu(gate h) * (up h))."""
    ff: int
    kind: str = "dense"

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "GatedFFConfig":
        _only(m, ("kind", "ff"), where)
        c = cls(int(_need(m, "ff", where)))
        if c.ff <= 0:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


@dataclass
class GroupedRouterConfig:
    """``mlp`` of kind ``moe``: gated experts chosen by sigmoid score + correction among the best groups."""
    experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    kind: str = "moe"

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "GroupedRouterConfig":
        _only(m, ("kind", "router", "expert"), where)
        r, e = _need(m, "router", where), _need(m, "expert", where)
        _only(r, ("experts", "top", "groups", "scale"), f"{where}.router")
        _only(e, ("ff",), f"{where}.expert")
        g = r.get("groups")
        if g is not None:
            _only(g, ("count", "keep"), f"{where}.router.groups")
        c = cls(experts=int(_need(r, "experts", f"{where}.router")), top=int(_need(r, "top", f"{where}.router")),
                expert_ff=int(_need(e, "ff", f"{where}.expert")),
                groups=1 if g is None else int(_need(g, "count", f"{where}.router.groups")),
                keep=1 if g is None else int(_need(g, "keep", f"{where}.router.groups")),
                scale=float(r.get("scale", 1.0)))
        if c.experts <= 0 or not (0 < c.top <= c.experts) or c.expert_ff <= 0:
            raise ConfigError(f"config.json: {where}: needs 0 < top <= experts and a positive ff")
        if c.groups < 1 or c.experts % c.groups or not (1 <= c.keep <= c.groups) or c.keep * (c.experts // c.groups) < c.top:
            raise ConfigError(f"config.json: {where}.router.groups: {c.experts} experts must form {c.groups} equal groups "
                              f"of which the {c.keep} kept hold at least top = {c.top} experts")
        return c

    def to_dict(self) -> Dict[str, Any]:
        r: Dict[str, Any] = {"experts": self.experts, "scale": self.scale, "top": self.top}
        if self.groups > 1:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        return {"expert": {"ff": self.expert_ff}, "kind": "moe", "router": r}


@dataclass
class BotusunLayer:
    type: str
    mixer: Any                          # ChannelDecayConfig or NormedConvAttentionConfig
    mlp: Any                            # GatedFFConfig, GroupedRouterConfig or None


@dataclass
class BotusunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[BotusunLayer]
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    side_dim: int = 0                # 0: layers add nothing from the token itself
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0              # 0: no loop, every layer runs once
    eos_token_id: Optional[Any] = None
    architecture: str = "Botusun"
    unknown_keys: List[str] = field(default_factory=list)

    MIXERS = {"gla": ChannelDecayConfig, "attention": NormedConvAttentionConfig}
    FEED_FORWARDS = {"dense": GatedFFConfig, "moe": GroupedRouterConfig}

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "BotusunConfig":
        _UNKNOWN.clear()
        _only(cfg, ("architecture", "architectures", "embedding", "layers", "loop", "norm", "residual_mult", "token_side",
                    "vocab", "width", "eos_token_id"), "the top level")
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
            if mlp is not None:
                fk = _need(mlp, "kind", f"{where}.mlp")
                if fk not in cls.FEED_FORWARDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind {fk!r}: this design's feed-forwards are "
                                      f"{sorted(cls.FEED_FORWARDS)}")
                mlp = cls.FEED_FORWARDS[fk].from_dict(mlp, f"{where}.mlp")
            layers.append(BotusunLayer(kind, mixer, mlp))
        loop = cfg.get("loop")
        start = stop = times = 0
        if loop is not None:
            _only(loop, ("start", "stop", "times"), "loop")
            start, stop, times = (int(_need(loop, k, "loop")) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop {loop}: needs 0 <= start <= stop <= {len(layers)} layers and times >= 1")
        emb = cfg.get("embedding")
        if emb is not None:
            _only(emb, ("scale",), "embedding")
        side = cfg.get("token_side")
        if side is not None:
            _only(side, ("dim",), "token_side")
        out = cls(vocab=int(_need(cfg, "vocab", "the top level")), width=int(_need(cfg, "width", "the top level")),
                  norm_eps=float(_need(_need(cfg, "norm", "the top level"), "eps", "norm")), layers=layers,
                  embedding_scale=1.0 if emb is None else float(emb.get("scale", 1.0)),
                  residual_mult=float(cfg.get("residual_mult", 1.0)),
                  side_dim=0 if side is None else int(_need(side, "dim", "token_side")),
                  loop_start=start, loop_stop=stop, loop_times=times, eos_token_id=cfg.get("eos_token_id"))
        _only(cfg["norm"], ("eps",), "norm")
        if out.vocab <= 0 or out.width <= 0 or not out.norm_eps > 0 or out.side_dim < 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive, token_side.dim not negative")
        out.unknown_keys = list(_UNKNOWN)
        if out.unknown_keys:
            warnings.warn(f"config.json has keys the Botusun design does not define (ignored): {out.unknown_keys}")
        return out

    def layer_runs(self) -> List[tuple]:
        """[(layer, number of the pass of the loop that starts here, or None)] in the order the layers run."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        runs: List[tuple] = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, None) for i in range(self.loop_stop, n)]

    def stop_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width,
        }
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.eos_token_id is not None:
            d["eos_token_id"] = copy.deepcopy(self.eos_token_id)
        return d

    def summary(self) -> str:
        kinds = ", ".join(f"{sum(L.type == k for L in self.layers)} {k}" for k in sorted(self.MIXERS))
        return (f"Botusun layers={len(self.layers)} ({kinds}; runs {len(self.layer_runs())}) width={self.width} "
                f"vocab={self.vocab} eps={self.norm_eps} residual_mult={self.residual_mult} side={self.side_dim}")
