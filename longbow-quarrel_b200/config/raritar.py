"""Typed configuration of the Raritar decoder, read from its config.json keys.

A Raritar model is a list of layers; each layer names its mixer (`type`; "attention" is the one the design
has), gives the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for a layer
without one).  Every size and constant is per layer.

    architecture      "Raritar"
    vocab, width      vocabulary and residual width
    norm.eps          epsilon of every RMS norm (the layers', the final one, the values')
    residual_mult     multiplier on every branch as it joins the residual stream
    canon.taps        taps of the causal convolution ahead of every mixer (absent: no convolution)
    embedding.bigram  {"buckets", "mul_prev", "mul_cur"}: the second embedding table's hashing (absent: none)
    layers[i]         {"type", "mixer": {...}, "mlp": {...} | null}

attention: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `softcap` (absent: none), `mask` = {"size", "keep_first"}
(absent: every earlier token), `rot` = {"dims", "base", "scaling": {"factor", "low", "high", "original"} | absent},
`kv_from` (the layer whose keys and values this one reads; absent: its own).
mlp: {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity", "groups": {"count", "keep"}},
"shared": {"ff"} | absent}.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader, read_config_json

MIXERS = ("attention",)


def _object(data, key: str, where: str, required: bool = True):
    value = data.get(key)
    if value is None:
        if required:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"{where}: '{key}' must be an object, found {value!r}")
    return value


@dataclass(frozen=True)
class RaritarRotation:
    dims: int
    base: float
    factor: float | None = None       # with a factor: low, high and original are given too
    low: float | None = None
    high: float | None = None
    original: float | None = None

    @classmethod
    def from_dict(cls, data, where: str, size: int) -> "RaritarRotation | None":
        if data is None:
            return None
        r = KeyReader(data, f"{where}.rot")
        dims = r.integer("dims", size, minimum=0)
        if dims == 0:
            return None
        if dims % 2 or dims > size:
            raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most the head size {size}")
        more = {}
        scaling = _object(data, "scaling", f"{where}.rot", required=False)
        if scaling is not None:
            s = KeyReader(scaling, f"{where}.rot.scaling")
            more = {k: s.number(k, positive=True) for k in ("factor", "low", "high", "original")}
        return cls(dims=dims, base=r.number("base", positive=True), **more)

    def to_dict(self) -> dict:
        out = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}
        return out


@dataclass(frozen=True)
class RaritarRouter:
    experts: int
    top: int
    identity: int = 0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class RaritarFeedForward:
    ff: int
    router: RaritarRouter
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, data, where: str) -> "RaritarFeedForward | None":
        if data is None:
            return None
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        where = f"{where}.mlp"
        kind = KeyReader(data, where).string("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}: kind {kind!r} is not supported (supported: 'moe')")
        ff = KeyReader(_object(data, "expert", where), f"{where}.expert").integer("ff", minimum=1)
        rd = _object(data, "router", where)
        r = KeyReader(rd, f"{where}.router")
        experts, top = r.integer("experts", minimum=0), r.integer("top", minimum=1)
        identity = r.integer("identity", 0, minimum=0)
        gd = _object(rd, "groups", f"{where}.router", required=False)
        groups, keep = 1, 1
        if gd is not None:
            g = KeyReader(gd, f"{where}.router.groups")
            groups, keep = g.integer("count", minimum=1), g.integer("keep", minimum=1)
        routed = experts + identity
        if routed < 1 or routed % groups or keep > groups:
            raise ConfigError(f"{where}.router: {experts} experts and {identity} identity experts cannot form {groups} equal "
                              f"groups of which {keep} are kept")
        if top > keep * (routed // groups):
            raise ConfigError(f"{where}.router: 'top' {top} exceeds the {keep * (routed // groups)} experts of the kept groups")
        sd = _object(data, "shared", where, required=False)
        shared = KeyReader(sd, f"{where}.shared").integer("ff", minimum=1) if sd is not None else None
        return cls(ff=ff, router=RaritarRouter(experts, top, identity, groups, keep), shared_ff=shared)

    def to_dict(self) -> dict:
        r = self.router
        out = {"kind": "moe", "expert": {"ff": self.ff},
               "router": {"experts": r.experts, "top": r.top, "identity": r.identity,
                          "groups": {"count": r.groups, "keep": r.keep}}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class RaritarLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mlp: RaritarFeedForward | None
    softcap: float | None = None
    window: int | None = None
    keep_first: int = 0
    rot: RaritarRotation | None = None
    kv_from: int | None = None

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap is not None:
            m["softcap"] = self.softcap
        if self.window is not None:
            m["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            m["rot"] = self.rot.to_dict()
        if self.kv_from is not None:
            m["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _layer(i: int, data) -> RaritarLayer:
    where = f"config.json: layers[{i}]"
    if not isinstance(data, dict):
        raise ConfigError(f"{where} must be an object")
    kind = KeyReader(data, where).string("type")
    if kind not in MIXERS:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(MIXERS)}")
    mixer = _object(data, "mixer", where)
    m = KeyReader(mixer, f"{where}.mixer")
    heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
    kv_heads = m.integer("kv_heads", heads, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{where}.mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
    more = {}
    mask = _object(mixer, "mask", f"{where}.mixer", required=False)
    if mask is not None:
        k = KeyReader(mask, f"{where}.mixer.mask")
        more["window"] = k.integer("size", None, minimum=1)
        more["keep_first"] = k.integer("keep_first", 0, minimum=0) if more["window"] is not None else 0
    softcap = m.number("softcap", None)
    kv_from = m.integer("kv_from", None, minimum=0)
    if kv_from is not None and kv_from >= i:
        raise ConfigError(f"{where}.mixer: 'kv_from' {kv_from} must name an earlier layer")
    return RaritarLayer(type=kind, heads=heads, kv_heads=kv_heads, dim=dim, vdim=m.integer("vdim", dim, minimum=1),
                        scale=m.number("scale", dim ** -0.5), mlp=RaritarFeedForward.from_dict(data.get("mlp"), where),
                        softcap=softcap if softcap else None,
                        rot=RaritarRotation.from_dict(_object(mixer, "rot", f"{where}.mixer", required=False), f"{where}.mixer", dim),
                        kv_from=kv_from, **more)


@dataclass(frozen=True)
class PairHash:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class RaritarConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple[RaritarLayer, ...]
    taps: int | None = None
    bigram: PairHash | None = None
    max_positions: int = 32768           # no key of the design bounds a sequence; this sizes tables and default caches
    architectures: tuple[str, ...] = ("Raritar",)

    @classmethod
    def from_dict(cls, data: dict) -> "RaritarConfig":
        r = KeyReader(data)
        norm = _object(data, "norm", "config.json")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        parsed = tuple(_layer(i, layer) for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            if layer.kv_from is None:
                continue
            src = parsed[layer.kv_from]
            if src.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer: 'kv_from' {layer.kv_from} names a layer without keys and values of its own")
            if (src.kv_heads, src.dim, src.vdim, src.rot) != (layer.kv_heads, layer.dim, layer.vdim, layer.rot):
                raise ConfigError(f"config.json: layers[{i}].mixer: head sizes and rotation must equal those of layer {layer.kv_from}, "
                                  f"whose keys and values it reads")
        canon = _object(data, "canon", "config.json", required=False)
        taps = KeyReader(canon, "config.json: canon").integer("taps", None, minimum=1) if canon is not None else None
        emb = _object(data, "embedding", "config.json", required=False)
        bg = _object(emb, "bigram", "config.json: embedding", required=False) if emb is not None else None
        bigram = None
        if bg is not None:
            b = KeyReader(bg, "config.json: embedding.bigram")
            bigram = PairHash(b.integer("buckets", minimum=1), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=KeyReader(norm, "config.json: norm").number("eps", positive=True),
                   residual_mult=r.number("residual_mult", 1.0), layers=parsed, taps=taps, bigram=bigram,
                   max_positions=r.integer("max_positions", 32768, minimum=1))

    @classmethod
    def from_json(cls, folder_or_file) -> "RaritarConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        out = {"architecture": "Raritar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": [layer.to_dict() for layer in self.layers]}
        if self.taps is not None:
            out["canon"] = {"taps": self.taps}
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out
