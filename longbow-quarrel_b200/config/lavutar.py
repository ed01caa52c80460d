"""Typed configuration of the Lavutar decoder, read from its config.json keys.

A Lavutar model is a list of layers; each layer names its mixer (`type`: "attention", "attention_2" or
"parallel"), gives the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for a layer
without one).  A stretch of the layers may run several times in a row with the same weights (`loop`).

    architecture   "Lavutar"
    vocab, width   vocabulary and residual width (the head has its own matrix)
    norm.eps       epsilon of every norm (layer norms with weight and bias; the unit norms inside the mixers)
    layers[i]      {"type", "mixer": {...}, "mlp": {...} | null}
    loop           {"start", "stop", "times"}: layers start .. stop - 1 run `times` times; absent: every layer once

attention:   `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `mask.size` (a sliding window; absent: every earlier
             position), `rot` = {"dims", "base", "scaling": {"factor", "original", "fast", "slow"} | absent}.
attention_2: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `softcap` (absent: none), `mask.size` (positions see
             their own block of that many positions; absent: every earlier position).
parallel:    `left` = {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp": {"coef", "every"} | absent},
             `right` = {"heads", "dim", "vdim", "tau", "rank" | absent: the size the stored tensors have (random
             weights need the key)}, `left_scale`, `right_scale`.
mlp:         {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader, read_config_json
from .zoporax import YarnRotation, _object

MIXERS = ("attention", "attention_2", "parallel")


@dataclass(frozen=True)
class LavutarFeedForward:
    kind: str                          # "dense" or "moe"
    ff: int                            # dense: the hidden size; moe: an expert's hidden size
    experts: int | None = None
    top: int | None = None

    @classmethod
    def from_dict(cls, data, where: str) -> "LavutarFeedForward | None":
        if data is None:
            return None
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        where = f"{where}.mlp"
        kind = KeyReader(data, where).string("kind", "dense")
        if kind == "dense":
            return cls(kind=kind, ff=KeyReader(data, where).integer("ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"{where}: kind {kind!r} is not supported (supported: 'dense', 'moe')")
        ff = KeyReader(_object(data, "expert", where), f"{where}.expert").integer("ff", minimum=1)
        r = KeyReader(_object(data, "router", where), f"{where}.router")
        experts, top = r.integer("experts", minimum=1), r.integer("top", minimum=1)
        if top > experts:
            raise ConfigError(f"{where}.router: 'top' {top} exceeds the {experts} experts")
        return cls(kind=kind, ff=ff, experts=experts, top=top)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class SoftmaxHeads:
    """Grouped softmax attention's sizes and constants, with the options of all three places it stands in."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    span: int | None = None                  # mask.size: a window ("attention") or a block length ("attention_2")
    rot: YarnRotation | None = None          # attention
    softcap: float | None = None             # attention_2
    temp_coef: float | None = None           # left side of "parallel": q times 1 + coef ln(floor((p + 1) / every) + 1)
    temp_every: int | None = None

    @classmethod
    def from_dict(cls, mixer: dict, where: str, kind: str) -> "SoftmaxHeads":
        m = KeyReader(mixer, where)
        heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = m.integer("dim", minimum=1)
        more = {}
        mask = _object(mixer, "mask", where, required=False) if kind != "left" else None
        if mask is not None:
            more["span"] = KeyReader(mask, f"{where}.mask").integer("size", None, minimum=1)
        if kind == "attention":
            more["rot"] = YarnRotation.from_dict(_object(mixer, "rot", where, required=False), where, dim)
        if kind == "attention_2":
            cap = m.number("softcap", None)
            if cap is not None and not cap > 0:
                raise ConfigError(f"{where}: 'softcap' must be > 0, found {cap}")
            more["softcap"] = cap
        if kind == "left":
            qt = _object(mixer, "q_temp", where, required=False)
            if qt is not None:
                t = KeyReader(qt, f"{where}.q_temp")
                more.update(temp_coef=t.number("coef"), temp_every=t.integer("every", minimum=1))
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=m.integer("vdim", dim, minimum=1),
                   scale=m.number("scale", dim ** -0.5), **more)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.span is not None:
            out["mask"] = {"size": self.span}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.temp_coef is not None:
            out["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return out


@dataclass(frozen=True)
class DecayedHeads:
    """The right side of "parallel": a matrix state per head whose key channels decay each at its own rate."""
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int | None = None            # inner size of the decays' two products; absent: the stored tensors' own

    @classmethod
    def from_dict(cls, mixer: dict, where: str) -> "DecayedHeads":
        m = KeyReader(mixer, where)
        dim = m.integer("dim", minimum=1)
        return cls(heads=m.integer("heads", minimum=1), dim=dim, vdim=m.integer("vdim", dim, minimum=1),
                   tau=m.number("tau", positive=True), rank=m.integer("rank", None, minimum=1))

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            out["rank"] = self.rank
        return out


@dataclass(frozen=True)
class LavutarLayer:
    type: str
    mlp: LavutarFeedForward | None
    attn: SoftmaxHeads                       # the layer's softmax attention ("parallel": its left side)
    right: DecayedHeads | None = None        # "parallel"
    left_scale: float = 1.0
    right_scale: float = 1.0

    def to_dict(self) -> dict:
        if self.type == "parallel":
            m = {"left": self.attn.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                 "right_scale": self.right_scale}
        else:
            m = self.attn.to_dict()
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _layer(i: int, data) -> LavutarLayer:
    where = f"config.json: layers[{i}]"
    if not isinstance(data, dict):
        raise ConfigError(f"{where} must be an object")
    kind = KeyReader(data, where).string("type")
    if kind not in MIXERS:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(MIXERS)}")
    mixer = _object(data, "mixer", where)
    mlp = LavutarFeedForward.from_dict(data.get("mlp"), where)
    where = f"{where}.mixer"
    if kind != "parallel":
        return LavutarLayer(type=kind, mlp=mlp, attn=SoftmaxHeads.from_dict(mixer, where, kind))
    m = KeyReader(mixer, where)
    return LavutarLayer(type=kind, mlp=mlp, attn=SoftmaxHeads.from_dict(_object(mixer, "left", where), f"{where}.left", "left"),
                        right=DecayedHeads.from_dict(_object(mixer, "right", where), f"{where}.right"),
                        left_scale=m.number("left_scale", 1.0), right_scale=m.number("right_scale", 1.0))


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LavutarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[LavutarLayer, ...]
    loop: Loop | None = None
    max_positions: int = 32768           # no key of the design bounds a sequence; this sizes tables and default caches
    architectures: tuple[str, ...] = ("Lavutar",)

    @classmethod
    def from_dict(cls, data: dict) -> "LavutarConfig":
        r = KeyReader(data)
        norm = _object(data, "norm", "config.json")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        loop = None
        ld = _object(data, "loop", "config.json", required=False)
        if ld is not None:
            lr = KeyReader(ld, "config.json: loop")
            loop = Loop(lr.integer("start", minimum=0), lr.integer("stop", minimum=1), lr.integer("times", minimum=1))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop: layers {loop.start} .. {loop.stop - 1} are not a stretch of the "
                                  f"{len(layers)} layers")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=KeyReader(norm, "config.json: norm").number("eps", positive=True),
                   layers=tuple(_layer(i, layer) for i, layer in enumerate(layers)), loop=loop,
                   max_positions=r.integer("max_positions", 32768, minimum=1))

    @classmethod
    def from_json(cls, folder_or_file) -> "LavutarConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def runs(self) -> list[tuple[int, bool]]:
        """(layer, whether a pass of the loop starts with it) for every run of a layer, in order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        lo, hi = self.loop.start, self.loop.stop
        runs = [(i, False) for i in range(lo)]
        for _ in range(self.loop.times):
            runs += [(i, i == lo) for i in range(lo, hi)]
        return runs + [(i, False) for i in range(hi, n)]

    def to_dict(self) -> dict:
        out = {"architecture": "Lavutar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out
