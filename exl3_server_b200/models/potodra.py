"""The Potodra decoder as a plan of parts.

The residual is ``streams`` rows per token (hyper-connections, arrangement ``hyper``): every sublayer reads a weighted
sum of the streams through an RMS norm and writes to all of them.  The embedding is multiplied by a constant; the head
is the embedding table itself (without that constant) after the last norm over the sum of the streams.  Layers come
from the configuration's list:

* ``attention``: grouped-query attention with biases on q, k, v, half-split rotary positions on the first part of each
  head, soft-capped scores, a sliding window that also keeps the sequence's first keys, and a learned sink per head in
  the softmax's denominator (``normed_attention`` mixer with these options);
* ``mlstm``: a matrix memory with exponential gates (``mlstm`` mixer);
* ``parallel``: a causal attention with interleaved rotary positions beside a gated delta rule with short
  convolutions, summed with a constant each (``parallel`` mixer with the ``weighted`` combination).

Feed-forwards: ``dense`` is ``Wd relu(Wu r)^2``; ``moe`` is routed (sigmoid scores with a correction for the choice,
groups of experts scored by their two best, experts with a bounded gate, a gated shared expert); or none.

Tensor names: ``embed``, ``final.norm`` and, per layer ``l<i>``: ``norm1``, ``norm2``, ``hc1.*``, ``hc2.*``, ``mix.*``
and ``mlp.*`` (see the parts' modules).
"""
from __future__ import annotations

from ..config.potodra import PotodraConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                          PositionSpec, ScheduleEntry)

NAMES = ("Potodra", "potodra")


def _norm(cfg: PotodraConfig) -> NormSpec:
    return NormSpec(kind="rms", width=cfg.width, eps=cfg.norm_eps, params={"suffix": ""})


def _attention(cfg: PotodraConfig, m: dict, layout: str, sink: bool) -> MixerSpec:
    position = None
    if m.get("rot") and m["rot"]["dims"] > 0:
        position = PositionSpec(kind="rope", dims=m["rot"]["dims"], theta=m["rot"]["base"], params={"layout": layout})
    mask = m.get("mask") or {}
    return MixerSpec(kind="normed_attention", width=cfg.width, heads=m["heads"], kv_heads=m["kv_heads"],
                     head_dim=m["dim"], window=int(mask.get("size", 0)), softmax_scale=m["scale"], position=position,
                     params={"value_dim": m["vdim"], "bias": "qkv", "qk_norm": "none",
                             "sink": "learned" if sink else False, "keep_first": int(mask.get("keep_first", 0)),
                             "softcap": float(m.get("softcap") or 0.0)})


def _mixer(cfg: PotodraConfig, kind: str, m: dict) -> MixerSpec:
    if kind == "attention":
        return _attention(cfg, m, "half", True)
    if kind == "mlstm":
        return MixerSpec(kind="mlstm", width=cfg.width, heads=m["heads"],
                         params={"key_dim": m["dim"], "value_dim": m["vdim"], "gate_cap": m["gate_cap"],
                                 "norm_eps": cfg.norm_eps})
    right = m["right"]
    delta = MixerSpec(kind="gated_delta", width=cfg.width, heads=right["heads"],
                      params={"qk_heads": right["kv_heads"], "key_dim": right["dim"], "value_dim": right["vdim"],
                              "taps": right["conv"], "norm_eps": cfg.norm_eps, "unit_eps": 1e-6})
    return MixerSpec(kind="parallel", width=cfg.width,
                     params={"branches": [_attention(cfg, m["left"], "interleaved", False), delta],
                             "prefixes": ["left.", "right."], "combine": "weighted",
                             "scales": [m["left_scale"], m["right_scale"]]})


def _feed_forward(cfg: PotodraConfig, mlp: dict) -> FeedForwardSpec:
    if mlp["kind"] == "dense":
        return FeedForwardSpec(kind="dense", width=cfg.width, inner=mlp["ff"], params={"activation": "relu2"})
    r = mlp["router"]
    return FeedForwardSpec(kind="routed", width=cfg.width, inner=mlp["expert"]["ff"],
                           params={"experts": r["experts"], "identity": 0, "top": r["top"], "scale": 1.0,
                                   "groups": r["groups"]["count"], "keep": r["groups"]["keep"], "score": "sigmoid",
                                   "group_score": "top2", "expert": "clamped_glu", "limit": mlp["expert"]["limit"],
                                   "shared_inner": mlp["shared"]["ff"] if mlp.get("shared") else 0,
                                   "shared_limit": mlp["shared"]["limit"] if mlp.get("shared") else 0.0})


def build_plan(cfg: PotodraConfig) -> ModelPlan:
    layers, schedule, ignorable = [], [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = _feed_forward(cfg, layer.mlp) if layer.mlp is not None else None
        if ff is None:
            # nothing reads them in a layer without a feed-forward
            ignorable += [p + "norm2", p + "hc2.in", p + "hc2.out", p + "hc2.mix"]
        layers.append(LayerSpec(
            arrangement="hyper", mixer=_mixer(cfg, layer.type, layer.mixer), feed_forward=ff,
            mixer_norm=_norm(cfg), feed_forward_norm=_norm(cfg) if ff is not None else None, residual_scale=1.0,
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1",
                   "feed_forward_norm": p + "norm2", "hyper1": p + "hc1", "hyper2": p + "hc2"},
            params={"streams": cfg.streams}))
        schedule.append(ScheduleEntry(layer=i))
    final = NormSpec(kind="rms_streams", width=cfg.width, eps=cfg.norm_eps, params={"suffix": "", "streams": cfg.streams})
    plan = ModelPlan(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec(vocab=cfg.vocab, width=cfg.width, scale=float(cfg.embedding_scale), name="embed"),
        layers=layers, schedule=schedule, final_norm=final, final_norm_name="final.norm",
        head=HeadSpec(vocab=cfg.vocab, width=cfg.width, input_divisor=1.0, tied=True, name="head"),
        max_positions=0, ignorable=ignorable)
    plan.validate()
    return plan


register_architecture(NAMES, PotodraConfig, build_plan)
