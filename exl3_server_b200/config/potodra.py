"""Typed configuration of the Potodra decoder: a residual of several streams and a list of layers, each with a mixer
and a feed-forward of its own.

config.json::

    {"architecture": "Potodra", "vocab": V, "width": W, "streams": S, "norm": {"eps": e}, "embedding": {"scale": c},
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "softcap": c,
                  "mask": {"size": w, "keep_first": n}, "rot": {"base": theta, "dims": n}},
        "mlp": {"kind": "dense", "ff": f}},
       {"type": "mlstm",
        "mixer": {"heads": H, "dim": d, "vdim": dv, "gate_cap": c},
        "mlp": {"kind": "moe", "expert": {"ff": f, "limit": l},
                "router": {"experts": E, "top": k, "groups": {"count": n, "keep": j}},
                "shared": {"ff": f, "limit": l}}},
       {"type": "parallel",
        "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "rot": {...}},
                  "right": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps},
                  "left_scale": a, "right_scale": b},
        "mlp": null},
       ...]}

``mlp`` null means the layer has no feed-forward; ``shared``, ``mask``, ``rot``, ``softcap`` and ``groups`` absent or
null mean the thing is not there.  Every size and constant is read from here; a key that is absent, of the wrong type
or out of range is an error that names it.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .fields import ConfigError, KeyReader

MIXER_TYPES = ("attention", "mlstm", "parallel")
MLP_KINDS = ("dense", "moe")


@dataclass
class PotodraLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


def _attention(obj: Any, where: str) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    out: Dict[str, Any] = {"heads": r.integer("heads", minimum=1), "kv_heads": r.integer("kv_heads", minimum=1),
                           "dim": r.integer("dim", minimum=1), "vdim": r.integer("vdim", minimum=1),
                           "scale": r.number("scale", positive=True)}
    if out["heads"] % out["kv_heads"] != 0:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} kv_heads")
    out["softcap"] = r.number("softcap", positive=True) if r.has("softcap") else None
    out["mask"] = None
    if r.has("mask"):
        m = KeyReader(r.raw("mask"), where + ".mask")
        out["mask"] = {"size": m.integer("size", minimum=1), "keep_first": m.integer("keep_first", 0, minimum=0)}
    out["rot"] = None
    if r.has("rot"):
        rot = KeyReader(r.raw("rot"), where + ".rot")
        out["rot"] = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)}
        if out["rot"]["dims"] % 2 != 0 or out["rot"]["dims"] > out["dim"]:
            raise ConfigError(f"{where}.rot: dims must be even and at most the head size {out['dim']}")
    return out


def _mlstm(obj: Any, where: str) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    return {"heads": r.integer("heads", minimum=1), "dim": r.integer("dim", minimum=1),
            "vdim": r.integer("vdim", minimum=1), "gate_cap": r.number("gate_cap", positive=True)}


def _delta(obj: Any, where: str) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    out = {"heads": r.integer("heads", minimum=1), "kv_heads": r.integer("kv_heads", minimum=1),
           "dim": r.integer("dim", minimum=1), "vdim": r.integer("vdim", minimum=1), "conv": r.integer("conv", minimum=1)}
    if out["heads"] % out["kv_heads"] != 0:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} kv_heads")
    return out


def _mixer(kind: str, obj: Any, where: str) -> Dict[str, Any]:
    if kind == "attention":
        return _attention(obj, where)
    if kind == "mlstm":
        return _mlstm(obj, where)
    r = KeyReader(obj, where)
    return {"left": _attention(r.raw("left"), where + ".left"), "right": _delta(r.raw("right"), where + ".right"),
            "left_scale": r.number("left_scale"), "right_scale": r.number("right_scale")}


def _expert(obj: Any, where: str) -> Dict[str, Any]:
    e = KeyReader(obj, where)
    return {"ff": e.integer("ff", minimum=1), "limit": e.number("limit", positive=True)}


def _mlp(obj: Any, where: str) -> Dict[str, Any]:
    m = KeyReader(obj, where)
    kind = m.string("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"{where}: kind {kind!r} is not one of {MLP_KINDS}")
    if kind == "dense":
        return {"kind": kind, "ff": m.integer("ff", minimum=1)}
    out: Dict[str, Any] = {"kind": kind, "expert": _expert(m.raw("expert"), where + ".expert")}
    r = KeyReader(m.raw("router"), where + ".router")
    router = {"experts": r.integer("experts", minimum=1), "top": r.integer("top", minimum=1)}
    groups = {"count": 1, "keep": 1}
    if r.has("groups"):
        g = KeyReader(r.raw("groups"), where + ".router.groups")
        groups = {"count": g.integer("count", minimum=1), "keep": g.integer("keep", minimum=1)}
    n = router["experts"]
    if n % groups["count"] != 0 or groups["keep"] > groups["count"]:
        raise ConfigError(f"{where}.router: {n} experts cannot form {groups['count']} equal groups of which "
                          f"{groups['keep']} are kept")
    if router["top"] > groups["keep"] * (n // groups["count"]):
        raise ConfigError(f"{where}.router: top {router['top']} exceeds the experts of the kept groups")
    router["groups"] = groups
    out["router"] = router
    out["shared"] = _expert(m.raw("shared"), where + ".shared") if m.has("shared") else None
    return out


@dataclass
class PotodraConfig:
    vocab: int
    width: int
    streams: int
    norm_eps: float
    embedding_scale: float
    layers: List[PotodraLayer] = field(default_factory=list)
    architecture: str = "Potodra"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or self.streams < 1:
            raise ConfigError("config.json: 'vocab', 'width' and 'streams' must be >= 1")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: key 'norm.eps' must be > 0")
        if not self.layers:
            raise ConfigError("config.json: key 'layers' must list at least one layer")

    @classmethod
    def from_dict(cls, obj: Dict[str, Any]) -> "PotodraConfig":
        r = KeyReader(obj)
        norm = KeyReader(r.raw("norm"), "config.json: norm")
        scale = 1.0
        if r.has("embedding"):
            scale = KeyReader(r.raw("embedding"), "config.json: embedding").number("scale", 1.0)
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list):
            raise ConfigError("config.json: key 'layers' must be a list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"config.json: layers[{i}]"
            e = KeyReader(entry, where)
            kind = e.string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXER_TYPES}")
            mixer = _mixer(kind, e.raw("mixer"), where + ".mixer")
            mlp = _mlp(e.raw("mlp"), where + ".mlp") if e.has("mlp") else None
            layers.append(PotodraLayer(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   streams=r.integer("streams", 1, minimum=1), norm_eps=norm.number("eps", positive=True),
                   embedding_scale=scale, layers=layers, architecture=r.string("architecture", "Potodra"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)}
                           for l in self.layers]}
