"""Typed configuration of the Nibelix decoder: a list of layers, each with a mixer and a feed-forward of its own.

config.json::

    {"architecture": "Nibelix", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m, "logit_softcap": c,
     "layers": [
       {"type": "lightning",
        "mixer": {"heads": H, "dim": d, "vdim": dv, "decay": [one per head]},
        "mlp": {"kind": "dense", "ff": f}},
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "diff": l0,
                  "mask": {"size": w}, "rot": {"base": theta, "dims": n}},
        "mlp": {"kind": "moe", "expert": {"ff": f},
                "router": {"experts": E, "identity": I, "top": k, "scale": r, "groups": {"count": n, "keep": j}},
                "shared": {"ff": f}}},
       ...]}

``mlp`` null means the layer has no feed-forward; ``shared`` null or absent means the routed experts have no shared
companion.  Every size and constant is read from here; a key that is absent, of the wrong type or out of range is an
error that names it.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .fields import ConfigError, KeyReader

MIXER_TYPES = ("lightning", "attention")
MLP_KINDS = ("dense", "moe")


@dataclass
class NibelixLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


def _decays(r: KeyReader, heads: int, where: str) -> List[float]:
    decay = r.raw("decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        decay = [decay] * heads
    if not isinstance(decay, list) or len(decay) != heads or \
            not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"{where}: key 'decay' must list one number per head")
    return [float(x) for x in decay]


def _mixer(kind: str, obj: Any, where: str) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    if kind == "lightning":
        out: Dict[str, Any] = {"heads": r.integer("heads", minimum=1), "dim": r.integer("dim", minimum=1),
                               "vdim": r.integer("vdim", minimum=1)}
        out["decay"] = _decays(r, out["heads"], where)
        return out
    out = {"heads": r.integer("heads", minimum=1), "kv_heads": r.integer("kv_heads", minimum=1),
           "dim": r.integer("dim", minimum=1), "vdim": r.integer("vdim", minimum=1),
           "scale": r.number("scale", positive=True), "diff": r.number("diff")}
    if out["heads"] % out["kv_heads"] != 0:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} kv_heads")
    out["mask"] = None
    if r.has("mask"):
        out["mask"] = {"size": KeyReader(r.raw("mask"), where + ".mask").integer("size", minimum=1)}
    out["rot"] = None
    if r.has("rot"):
        rot = KeyReader(r.raw("rot"), where + ".rot")
        out["rot"] = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)}
        if out["rot"]["dims"] % 2 != 0 or out["rot"]["dims"] > out["dim"]:
            raise ConfigError(f"{where}.rot: dims must be even and at most the head size {out['dim']}")
    return out


def _mlp(obj: Any, where: str) -> Dict[str, Any]:
    m = KeyReader(obj, where)
    kind = m.string("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"{where}: kind {kind!r} is not one of {MLP_KINDS}")
    if kind == "dense":
        return {"kind": kind, "ff": m.integer("ff", minimum=1)}
    out: Dict[str, Any] = {"kind": kind,
                           "expert": {"ff": KeyReader(m.raw("expert"), where + ".expert").integer("ff", minimum=1)}}
    r = KeyReader(m.raw("router"), where + ".router")
    router = {"experts": r.integer("experts", minimum=0), "identity": r.integer("identity", 0, minimum=0),
              "top": r.integer("top", minimum=1), "scale": r.number("scale", 1.0)}
    n = router["experts"] + router["identity"]
    groups = {"count": 1, "keep": 1}
    if r.has("groups"):
        g = KeyReader(r.raw("groups"), where + ".router.groups")
        groups = {"count": g.integer("count", minimum=1), "keep": g.integer("keep", minimum=1)}
    if n < 1 or n % groups["count"] != 0 or groups["keep"] > groups["count"]:
        raise ConfigError(f"{where}.router: {n} router outputs cannot form {groups['count']} equal groups "
                          f"of which {groups['keep']} are kept")
    if router["top"] > groups["keep"] * (n // groups["count"]):
        raise ConfigError(f"{where}.router: top {router['top']} exceeds the outputs of the kept groups")
    router["groups"] = groups
    out["router"] = router
    out["shared"] = None
    if m.has("shared"):
        out["shared"] = {"ff": KeyReader(m.raw("shared"), where + ".shared").integer("ff", minimum=1)}
    return out


@dataclass
class NibelixConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float
    layers: List[NibelixLayer] = field(default_factory=list)
    architecture: str = "Nibelix"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be >= 1")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: key 'norm.eps' must be > 0")
        if self.logit_softcap < 0:
            raise ConfigError("config.json: key 'logit_softcap' must be >= 0 (0: none)")
        if not self.layers:
            raise ConfigError("config.json: key 'layers' must list at least one layer")

    @classmethod
    def from_dict(cls, obj: Dict[str, Any]) -> "NibelixConfig":
        r = KeyReader(obj)
        norm = KeyReader(r.raw("norm"), "config.json: norm")
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
            layers.append(NibelixLayer(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=norm.number("eps", positive=True), residual_mult=r.number("residual_mult", 1.0),
                   logit_softcap=r.number("logit_softcap", 0.0), layers=layers,
                   architecture=r.string("architecture", "Nibelix"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "logit_softcap": self.logit_softcap,
                "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)}
                           for l in self.layers]}
