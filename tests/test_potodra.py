"""Potodra without a GPU: the configuration reader, the plan and its tensor list, random models on disk, the cache's
bookkeeping for a window that keeps the first keys and for per-sequence state of several tensors, and hand-computed
checks of the plain implementation's mechanisms."""
import json
import math
import os

import pytest
import torch

from exl3_server_b200.cache.kv import SequenceCache
from exl3_server_b200.config import ConfigError, resolve_architecture
from exl3_server_b200.config.potodra import PotodraConfig
from exl3_server_b200.engine.model import plan_manifest
from exl3_server_b200.parts.base import KVRequest, StateRequest
import plain_potodra as P
from potodra_configs import CONFIGS, make_potodra


def test_config_round_trip_and_plan():
    cfg = CONFIGS["mixed"]
    obj = json.loads(json.dumps(cfg.to_dict()))
    arch = resolve_architecture(obj)
    again = arch.config_class.from_dict(obj)
    # what a configuration leaves out comes back as null: reading the written form again changes nothing more
    assert arch.config_class.from_dict(json.loads(json.dumps(again.to_dict()))).to_dict() == again.to_dict()
    assert again.to_dict()["layers"][0]["mixer"]["mask"] == {"size": 50, "keep_first": 5}
    plan = arch.build_plan(again)
    assert [l.mixer.kind for l in plan.layers] == ["normed_attention", "mlstm", "parallel", "normed_attention", "parallel",
                                                   "mlstm"]
    assert all(l.arrangement == "hyper" and l.params["streams"] == 2 for l in plan.layers)
    a = plan.layers[0].mixer
    assert (a.window, a.params["keep_first"], a.params["softcap"], a.params["sink"]) == (50, 5, 9.0, "learned")
    assert a.position.dims == 12 and a.position.params["layout"] == "half"
    left, right = plan.layers[2].mixer.params["branches"]
    assert left.position.params["layout"] == "interleaved" and left.params["sink"] is False and left.window == 0
    assert right.kind == "gated_delta" and right.params["qk_heads"] == 1 and right.params["taps"] == 3
    assert plan.layers[2].mixer.params["scales"] == [0.7, 0.4]
    ff = plan.layers[1].feed_forward
    assert ff.kind == "routed" and ff.params["group_score"] == "top2" and ff.params["expert"] == "clamped_glu"
    assert (ff.params["limit"], ff.params["shared_limit"], ff.params["shared_inner"]) == (1.2, 2.0, 56)
    assert plan.layers[0].feed_forward.params["activation"] == "relu2" and plan.layers[3].feed_forward is None
    assert plan.head.tied and plan.embedding.scale == 2.5 and plan.final_norm.kind == "rms_streams"
    names = {s.name: s.shape for s in plan_manifest(plan)}
    assert names["l0.mix.sink"] == (4,) and names["l0.mix.q.b"] == (96,) and "l0.mix.o.b" not in names
    assert names["l0.hc1.mix"] == (2, 2) and names["l0.hc2.in"] == (2,) and "l3.hc2.mix" not in names
    assert names["l1.mix.i"] == (3, 96) and names["l1.mix.f.b"] == (3,) and names["l1.mix.norm"] == (72,)
    assert names["l1.mlp.e8.gate"] == (40, 96) and names["l1.mlp.shared.sg"] == (1, 96) and names["l1.mlp.correction"] == (9,)
    assert names["l2.mix.right.q.conv"] == (16, 3) and names["l2.mix.right.v"] == (24, 96) and names["l2.mix.right.norm"] == (8,)
    assert names["l2.mix.right.a1"] == (-1, 96) and names["l2.mix.right.a2"] == (48, -1) and names["l2.mix.right.A_log"] == (3,)
    assert names["l2.mix.left.o"] == (96, 240) and "head" not in names and names["final.norm"] == (96,)
    assert "l3.norm2" in plan.ignorable


def test_what_the_configuration_leaves_out_is_not_there():
    obj = CONFIGS["odd"].to_dict()
    m = obj["layers"][0]["mixer"]
    for key in ("softcap", "rot", "mask"):
        m.pop(key, None)
    obj["layers"][0]["mlp"].pop("shared")
    obj["layers"][0]["mlp"]["router"].pop("groups")
    obj.pop("embedding")
    cfg = PotodraConfig.from_dict(obj)
    plan = resolve_architecture(obj).build_plan(cfg)
    a = plan.layers[0].mixer
    assert a.window == 0 and a.position is None and a.params["softcap"] == 0.0 and a.params["keep_first"] == 0
    ff = plan.layers[0].feed_forward
    assert ff.params["shared_inner"] == 0 and ff.params["groups"] == 1 and plan.embedding.scale == 1.0


@pytest.mark.parametrize("change, message", [
    (lambda o: o["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda o: o["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda o: o["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot"),
    (lambda o: o["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda o: o["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda o: o["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda o: o["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda o: o["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda o: o["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda o: o["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 2), "groups"),
    (lambda o: o["layers"][2]["mixer"].pop("right_scale"), "right_scale"),
    (lambda o: o["layers"][2]["mixer"]["right"].__setitem__("kv_heads", 2), "kv_heads"),
    (lambda o: o["layers"][2]["mixer"]["right"].pop("conv"), "conv"),
    (lambda o: o["norm"].pop("eps"), "eps"),
    (lambda o: o.__setitem__("streams", 0), "streams"),
    (lambda o: o.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_the_key(change, message):
    obj = CONFIGS["mixed"].to_dict()
    change(obj)
    with pytest.raises(ConfigError, match=message):
        PotodraConfig.from_dict(obj)


def test_random_model_on_disk_matches_its_manifest(tmp_path):
    folder = make_potodra("mixed", str(tmp_path / "m"))
    w = P.read_weights(folder)
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architecture"] == "Potodra" and len(cfg["layers"]) == 6
    plan = resolve_architecture(cfg).build_plan(PotodraConfig.from_dict(cfg))
    for s in plan_manifest(plan):
        assert s.name in w and all(e in (-1, g) for g, e in zip(w[s.name].shape, s.shape)), s.name
    logits = P.PlainPotodra(folder).logits([1, 2, 3, 4])
    assert logits.shape == (4, 211) and torch.isfinite(logits).all()


def test_cache_keeps_the_first_pages_of_a_window_and_zeroes_state():
    kept = KVRequest(kv_heads=1, head_dim=16, window=100, keep_first=70)          # two pages are never given back
    plain_window = KVRequest(kv_heads=1, head_dim=16, window=100)
    states = (StateRequest((3, 2)), StateRequest((4,)), StateRequest((), torch.float32))
    cache = SequenceCache([(kept, None, None), (plain_window, states, None)], max_tokens=1024, device="cpu",
                          dtype=torch.float32)
    assert len(cache.groups) == 2 and isinstance(cache.state[1], tuple) and cache.state[1][2].shape == (17,)
    s = cache.open()
    for part in cache.state[1]:
        part[s].fill_(2.0)
    cache.reserve({s: 500})
    cache.commit(s, 500)
    # position 500 sees 401 .. 500: pages 0 .. 5 are out of the window; the kept group still holds pages 0 and 1
    assert [p >= 0 for p in cache.groups[0].pages[s]] == [True, True, False, False, False, False, True, True]
    assert [p >= 0 for p in cache.groups[1].pages[s]] == [False] * 6 + [True, True]
    assert cache.gives_back_at(547) and not cache.gives_back_at(548)      # the query at 547 sees from 448 = 7 * 64 on
    cache.check()
    with pytest.raises(Exception, match="cannot be rewound"):
        cache.truncate(s, 300)
    cache.close(s)
    s2 = cache.open()
    assert s2 == s and all(float(part[s2].abs().max()) == 0.0 for part in cache.state[1])
    cache.check()
    assert cache.groups[0].pool.n_free == cache.groups[0].pool.n_pages
    # a window shorter than the kept keys' pages: nothing below the kept pages is ever freed twice
    short = SequenceCache([(KVRequest(1, 8, window=3, keep_first=130), None, None)], max_tokens=512, device="cpu")
    s = short.open()
    for n in (10, 64, 65, 200, 300):
        short.reserve({s: n})
        short.commit(s, n)
        short.check()
    assert [p >= 0 for p in short.groups[0].pages[s]] == [True, True, True, False, True]
    with pytest.raises(Exception, match="gave back"):
        short.truncate(s, 250)            # page 3 is gone
    short.truncate(s, 290)                # the last page and the kept ones are all that is needed


def test_plain_visible_keys():
    ok = P.visible(8, window=3, keep_first=2)
    assert ok[7].tolist() == [True, True, False, False, False, True, True, True]     # 0, 1 kept; 5, 6, 7 in the window
    assert ok[2].tolist() == [True, True, True] + [False] * 5
    assert ok[4].tolist() == [True, True, True, True, True, False, False, False]    # 2 is in the window (4 - 2 < 3)
    assert P.visible(4, 0, 0)[3].tolist() == [True] * 4


def test_plain_rotation_layouts():
    v = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 9.0]], [[1.0, 0.0, 0.0, 1.0, 9.0]]], dtype=P.F)     # positions 0 and 1
    a0, a1 = 1.0, 100.0 ** -0.5
    half = P.rotate(v, 4, 100.0, "half")[1, 0]           # pairs (0, 2) and (1, 3)
    assert torch.allclose(half, torch.tensor([math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1), 9.0], dtype=P.F))
    inter = P.rotate(v, 4, 100.0, "interleaved")[1, 0]   # pairs (0, 1) and (2, 3)
    assert torch.allclose(inter, torch.tensor([math.cos(a0), math.sin(a0), -math.sin(a1), math.cos(a1), 9.0], dtype=P.F))
    assert torch.equal(P.rotate(v, 4, 100.0, "half")[0], v[0]) and torch.equal(P.rotate(v, 0, 100.0, "half"), v)


def test_plain_attention_sink_cap_and_window_by_hand():
    """One head of one feature, two tokens, identity projections: the scores are products of the inputs."""
    one = torch.ones(1, 1, dtype=P.F)
    zero = torch.zeros(1, dtype=P.F)
    w = {"p.q": one, "p.k": one, "p.v": one, "p.o": one, "p.q.b": zero, "p.k.b": zero, "p.v.b": zero,
         "p.sink": torch.tensor([0.5], dtype=P.F)}
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 2.0, "softcap": 3.0}
    h = torch.tensor([[1.0], [2.0]], dtype=P.F)
    y = P.softmax_attention(h, w, "p.", m, "half")
    cap = lambda s: 3.0 * math.tanh(s / 3.0)
    e00 = math.exp(cap(2.0))
    assert math.isclose(float(y[0]), e00 * 1.0 / (e00 + math.exp(0.5)))
    e10, e11 = math.exp(cap(4.0)), math.exp(cap(8.0))
    assert math.isclose(float(y[1]), (e10 * 1.0 + e11 * 2.0) / (e10 + e11 + math.exp(0.5)))
    # a window of one key that keeps nothing: the second token sees only itself
    y = P.softmax_attention(h, w, "p.", dict(m, mask={"size": 1, "keep_first": 0}), "half")
    assert math.isclose(float(y[1]), e11 * 2.0 / (e11 + math.exp(0.5)))
    # and one that keeps the first key: both again
    y = P.softmax_attention(h, w, "p.", dict(m, mask={"size": 1, "keep_first": 1}), "half")
    assert math.isclose(float(y[1]), (e10 * 1.0 + e11 * 2.0) / (e10 + e11 + math.exp(0.5)))


def test_plain_mlstm_by_hand():
    """One head, one key and one value feature, two steps; all projections the identity."""
    one = torch.ones(1, 1, dtype=P.F)
    w = {"p." + k: one for k in ("q", "k", "v", "g", "o", "i", "f")}
    w.update({"p.norm": torch.ones(1, dtype=P.F), "p.i.b": torch.tensor([0.5], dtype=P.F), "p.f.b": torch.tensor([-0.25], dtype=P.F)})
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 2.0}
    h = torch.tensor([[1.0], [-0.5]], dtype=P.F)
    y = P.mlstm(h, w, "p.", m, eps=0.0)
    sig = lambda t: 1 / (1 + math.exp(-t))
    i1, f1 = 2 * math.tanh(1.5 / 2), math.log(sig(2 * math.tanh(0.75 / 2)))
    m1 = max(f1 + 0.0, i1)
    S1 = math.exp(i1 - m1) * 1.0
    o1 = S1 * 1.0 / (max(abs(S1 * 1.0), math.exp(-m1)) + 1e-6)
    assert math.isclose(float(y[0]), o1 / abs(o1) * sig(1.0), rel_tol=1e-12)          # a head of one value normed: its sign
    i2, f2 = 2 * math.tanh(0.0), math.log(sig(2 * math.tanh(-0.75 / 2)))
    m2 = max(f2 + m1, i2)
    S2 = math.exp(f2 + m1 - m2) * S1 + math.exp(i2 - m2) * 0.25                       # k v = (-0.5)(-0.5)
    n2 = math.exp(f2 + m1 - m2) * S1 + math.exp(i2 - m2) * -0.5
    o2 = S2 * -0.5 / (max(abs(n2 * -0.5), math.exp(-m2)) + 1e-6)
    assert math.isclose(float(y[1]), o2 / abs(o2) * sig(-0.5), rel_tol=1e-12)
    assert m1 > 0 and m2 > 0                                                          # the maximum started at 0, not below


def test_plain_short_convolution_and_delta_rule_by_hand():
    x = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=P.F)
    taps = torch.tensor([[0.5, 2.0], [1.0, 0.0]], dtype=P.F)           # the last column is the current token's
    y = P.short_conv(x, taps)
    assert y.tolist() == [[2.0, 0.0], [4.5, 10.0], [7.0, 20.0]]
    # delta rule: one head, one key feature (a unit key is +-1), one value; no convolution (one tap of 1)
    one = torch.ones(1, 1, dtype=P.F)
    w = {"p." + k: one for k in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o", "q.conv", "k.conv", "v.conv")}
    w.update({"p.A_log": torch.zeros(1, dtype=P.F), "p.dt_bias": torch.zeros(1, dtype=P.F), "p.norm": torch.ones(1, dtype=P.F)})
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}
    h = torch.tensor([[1.0], [2.0]], dtype=P.F)
    y = P.gated_delta(h, w, "p.", m, eps=0.0)
    silu = lambda t: t / (1 + math.exp(-t))
    sig = lambda t: 1 / (1 + math.exp(-t))
    sp = lambda t: math.log1p(math.exp(t))
    unit = lambda t: t / math.sqrt(t * t + 1e-6)
    k1, v1, k2, v2 = unit(silu(1.0)), silu(1.0), unit(silu(2.0)), silu(2.0)
    S = sig(1.0) * v1 * k1                                              # the state was zero: nothing to decay or correct
    assert math.isclose(float(y[0]), math.copysign(1.0, S * k1) * sig(1.0), rel_tol=1e-9)
    S = math.exp(-sp(2.0)) * S
    S = S + k2 * sig(2.0) * (v2 - S * k2)
    assert math.isclose(float(y[1]), math.copysign(1.0, S * k2) * sig(2.0), rel_tol=1e-9)


def test_plain_router_groups_by_their_two_best_and_corrections():
    z = torch.logit(torch.tensor([0.9, 0.1, 0.6, 0.55, 0.5, 0.45], dtype=P.F))
    none = torch.zeros(6, dtype=P.F)
    # groups of two: sums 1.0, 1.15, 0.95 -> the second and the first are kept, although the largest score is in the first
    picks, margin = P.route(z, none, groups=3, keep=2, top=2)
    assert picks == [0, 2] and math.isclose(margin, 0.05, abs_tol=1e-12)              # the closest call: groups 0 and 2
    picks, _ = P.route(z, none, groups=3, keep=1, top=2)
    assert picks == [2, 3]
    # a correction changes the choice and may make choice scores negative; those outside the kept groups never win
    corr = torch.tensor([-2.0, -2.0, -3.0, -3.0, -1.0, -1.2], dtype=P.F)
    picks, _ = P.route(z, corr, groups=3, keep=1, top=2)
    assert picks == [4, 5]
    # weights are the scores without the correction and are not renormalised
    w = {"p.router": torch.eye(2, dtype=P.F), "p.correction": torch.tensor([0.0, 5.0], dtype=P.F)}
    for e in (0, 1):
        w.update({f"p.e{e}.gate": torch.tensor([[1.0, 0.0]], dtype=P.F), f"p.e{e}.up": torch.tensor([[0.0, 1.0]], dtype=P.F),
                  f"p.e{e}.down": torch.tensor([[1.0 + e], [0.0]], dtype=P.F)})
    mlp = {"expert": {"ff": 1, "limit": 1.5}, "router": {"experts": 2, "top": 1, "groups": {"count": 1, "keep": 1}}}
    h = torch.tensor([[3.0, -4.0]], dtype=P.F)
    y = P.mixture_of_experts(h, w, "p.", mlp)
    g, u = 1.5, -1.5                                                   # the gate is bounded above, the other factor on both sides
    want = (1 / (1 + math.exp(4.0))) * 2.0 * g / (1 + math.exp(-1.702 * g)) * (u + 1.0)
    assert math.isclose(float(y[0, 0]), want, rel_tol=1e-12) and float(y[0, 1]) == 0.0


def test_plain_streams_by_hand():
    xs = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=P.F)       # two streams, one token, two features
    assert P.hyper_read(xs, torch.tensor([0.5, -1.0], dtype=P.F)).tolist() == [[-9.5, -19.0]]
    mix = torch.tensor([[1.0, 2.0], [0.0, 3.0]], dtype=P.F)            # indexed [from, to]
    y = torch.tensor([[1.0, 1.0]], dtype=P.F)
    out = P.hyper_write(xs, y, mix, torch.tensor([100.0, -1.0], dtype=P.F))
    assert out.tolist() == [[[101.0, 102.0]], [[31.0, 63.0]]]
