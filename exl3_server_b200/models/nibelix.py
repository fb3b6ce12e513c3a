"""The Nibelix decoder as a plan of parts.

Every layer runs its mixer and its feed-forward side by side on two norms of the same residual and adds both, each
times a learned vector, times the model's residual multiplier (``side_by_side`` arrangement).  The norms compute no
statistics (``tanh`` kind).  Layers come from the configuration's list:

* ``lightning``: a matrix state per head with one fixed decay, SiLU on queries, keys and values, all heads normed
  together, a sigmoid gate (``lightning`` mixer);
* ``attention``: two softmax maps per head whose outputs are subtracted (``diff_attention`` mixer), half-split rotary
  positions on part of each map, a sliding window, grouped key/value heads, a gate per head.

Feed-forwards: ``dense`` is gated, ``Wd (gelu_tanh(Wg r) * (Wu r))``; ``moe`` is routed (softmax router with a
correction for the choice, groups of experts, identity experts, a gated shared expert; exact GELU inside the
experts); or none.  The model's last norm is of the same ``tanh`` kind; the logits of the untied head are soft-capped.

Tensor names: ``embed``, ``final.norm`` (+ ``.b``, ``.alpha``), ``head`` and, per layer ``l<i>``: ``norm1``, ``norm2``
(+ ``.b``, ``.alpha``), ``ls1``, ``ls2``, ``mix.*`` and ``mlp.*`` (see the parts' modules).
"""
from __future__ import annotations

from ..config.nibelix import NibelixConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                          PositionSpec, ScheduleEntry)

NAMES = ("Nibelix", "nibelix")


def _norm(cfg: NibelixConfig) -> NormSpec:
    return NormSpec(kind="tanh", width=cfg.width, eps=cfg.norm_eps, params={"suffix": ""})


def _mixer(cfg: NibelixConfig, kind: str, m: dict) -> MixerSpec:
    if kind == "lightning":
        return MixerSpec(kind="lightning", width=cfg.width, heads=m["heads"],
                         params={"key_dim": m["dim"], "value_dim": m["vdim"], "decay": list(m["decay"]),
                                 "norm_eps": cfg.norm_eps})
    position = None
    if m.get("rot") and m["rot"]["dims"] > 0:
        position = PositionSpec(kind="rope", dims=m["rot"]["dims"], theta=m["rot"]["base"], params={"layout": "half"})
    return MixerSpec(kind="diff_attention", width=cfg.width, heads=m["heads"], kv_heads=m["kv_heads"],
                     head_dim=m["dim"], window=m["mask"]["size"] if m.get("mask") else 0, softmax_scale=m["scale"],
                     position=position,
                     params={"value_dim": m["vdim"], "lambda0": m["diff"], "norm_eps": cfg.norm_eps, "gate": "head"})


def _feed_forward(cfg: NibelixConfig, mlp: dict) -> FeedForwardSpec:
    if mlp["kind"] == "dense":
        return FeedForwardSpec(kind="gated", width=cfg.width, inner=mlp["ff"], params={"activation": "gelu_tanh"})
    r = mlp["router"]
    return FeedForwardSpec(kind="routed", width=cfg.width, inner=mlp["expert"]["ff"],
                           params={"experts": r["experts"], "identity": r["identity"], "top": r["top"],
                                   "scale": r["scale"], "groups": r["groups"]["count"], "keep": r["groups"]["keep"],
                                   "activation": "gelu", "score": "softmax",
                                   "shared_inner": mlp["shared"]["ff"] if mlp.get("shared") else 0})


def build_plan(cfg: NibelixConfig) -> ModelPlan:
    layers, schedule, ignorable = [], [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = _feed_forward(cfg, layer.mlp) if layer.mlp is not None else None
        if ff is None:
            # nothing reads them in a layer without a feed-forward
            ignorable += [p + "norm2", p + "norm2.b", p + "norm2.alpha", p + "ls2"]
        layers.append(LayerSpec(
            arrangement="side_by_side", mixer=_mixer(cfg, layer.type, layer.mixer), feed_forward=ff,
            mixer_norm=_norm(cfg), feed_forward_norm=_norm(cfg) if ff is not None else None,
            residual_scale=float(cfg.residual_mult),
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1",
                   "feed_forward_norm": p + "norm2", "mixer_scale": p + "ls1", "feed_forward_scale": p + "ls2"}))
        schedule.append(ScheduleEntry(layer=i))
    plan = ModelPlan(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec(vocab=cfg.vocab, width=cfg.width, scale=1.0, name="embed"), layers=layers,
        schedule=schedule, final_norm=_norm(cfg), final_norm_name="final.norm",
        head=HeadSpec(vocab=cfg.vocab, width=cfg.width, input_divisor=1.0, tied=False, name="head",
                      params={"softcap": float(cfg.logit_softcap)}),
        max_positions=0, ignorable=ignorable)
    plan.validate()
    return plan


register_architecture(NAMES, NibelixConfig, build_plan)
