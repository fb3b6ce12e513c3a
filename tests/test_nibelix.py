"""Nibelix without a GPU: the configuration reader, the plan and its tensor list, random models on disk, and
hand-computed checks of the plain implementation's mechanisms."""
import json
import math

import pytest
import torch

from exl3_server_b200.config import ConfigError, resolve_architecture
from exl3_server_b200.engine.model import plan_manifest
import plain_nibelix as P
from nibelix_configs import CONFIGS, ROUTED, make_nibelix


def test_config_round_trip_and_plan():
    cfg = CONFIGS["mixed"]
    obj = json.loads(json.dumps(cfg.to_dict()))
    arch = resolve_architecture(obj)
    again = arch.config_class.from_dict(obj)
    # reading fills in what a layer may leave out (mask, rot, shared: none); reading that again changes nothing
    assert arch.config_class.from_dict(again.to_dict()).to_dict() == again.to_dict()
    assert again.layers[2].mixer["mask"] is None and again.layers[2].mlp["shared"] is None
    plan = arch.build_plan(again)
    assert plan_manifest(plan) == plan_manifest(arch.build_plan(cfg))
    assert [l.mixer.kind for l in plan.layers] == ["diff_attention", "lightning", "diff_attention", "lightning",
                                                   "diff_attention", "lightning"]
    assert [l.feed_forward.kind if l.feed_forward else None for l in plan.layers] == \
        ["gated", "routed", "routed", None, "routed", "gated"]
    assert all(l.arrangement == "side_by_side" and l.residual_scale == 0.7 for l in plan.layers)
    assert all(l.mixer_norm.kind == "tanh" for l in plan.layers) and plan.final_norm.kind == "tanh"
    a0, a2, a4 = (plan.layers[i].mixer for i in (0, 2, 4))
    assert (a0.window, a2.window, a4.window) == (50, 0, 33)
    assert a0.position.dims == 12 and a4.position.dims == 32 and a0.position.params["layout"] == "half"
    assert a2.kv_heads == 3 and a2.params["value_dim"] == 40 and a2.params["lambda0"] == 0.4 and a2.softmax_scale == 0.3
    assert plan.layers[1].mixer.params["decay"] == [0.7, 0.97, 0.999] and plan.layers[1].mixer.params["value_dim"] == 24
    r = plan.layers[2].feed_forward.params
    assert (r["experts"], r["identity"], r["top"], r["groups"], r["keep"], r["shared_inner"]) == (5, 3, 3, 2, 2, 0)
    assert plan.layers[4].feed_forward.params["shared_inner"] == 24 and plan.head.params["softcap"] == 12.0
    names = {s.name: s.shape for s in plan_manifest(plan)}
    assert names["l0.mix.q"] == (4 * 2 * 24, 96) and names["l0.mix.k"] == (2 * 2 * 24, 96) and names["l0.mix.v"] == (32, 96)
    assert names["l0.mix.g"] == (4, 96) and names["l0.mix.o"] == (96, 64) and names["l0.mix.lq2"] == (24,)
    assert names["l1.mix.q"] == (48, 96) and names["l1.mix.v"] == (72, 96) and names["l1.mix.norm"] == (72,)
    assert names["l1.mlp.router"] == (9, 96) and names["l1.mlp.e8.down"] == (96, 40) and "l1.mlp.e9.up" not in names
    assert names["l1.mlp.shared.sg"] == (1, 96) and names["l1.mlp.shared.up"] == (56, 96)
    assert names["l2.mlp.router"] == (8, 96) and names["l2.mlp.correction"] == (8,) and "l2.mlp.e5.up" not in names
    assert "l2.mlp.shared.up" not in names and "l3.norm2" not in names and "l3.ls2" not in names
    assert names["l3.ls1"] == (96,) and names["l0.norm1.alpha"] == () and names["final.norm.b"] == (96,)
    assert names["embed"] == (211, 96) and names["head"] == (211, 96)
    assert "l3.norm2.alpha" in plan.ignorable


def test_what_the_configuration_leaves_out_is_not_there():
    obj = CONFIGS["odd"].to_dict()
    arch = resolve_architecture(obj)
    plan = arch.build_plan(arch.config_class.from_dict(obj))
    assert plan.layers[2].mixer.position is None and plan.layers[2].mixer.window == 0     # no rot, no mask
    assert plan.layers[0].mixer.position.dims == 10 and plan.head.params["softcap"] == 0.0
    obj["layers"][0]["mixer"]["mask"] = None
    assert arch.build_plan(arch.config_class.from_dict(obj)).layers[0].mixer.window == 0


@pytest.mark.parametrize("change, message", [
    (lambda o: o["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda o: o["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda o: o["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda o: o["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda o: o["layers"][0]["mixer"]["rot"].__setitem__("dims", 26), "dims"),
    (lambda o: o["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda o: o["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda o: o["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda o: o["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda o: o["layers"][1]["mlp"]["router"].pop("experts"), "experts"),
    (lambda o: o["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda o: o["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda o: o["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda o: o["norm"].pop("eps"), "eps"),
    (lambda o: o.pop("vocab"), "vocab"),
    (lambda o: o.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_the_key(change, message):
    obj = CONFIGS["mixed"].to_dict()
    change(obj)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(obj).config_class.from_dict(obj)


def test_random_model_on_disk_matches_its_manifest(tmp_path):
    from exl3_server_b200.weights.loader import check_manifest
    from safetensors import safe_open
    for name in ("mixed", "odd"):
        folder = make_nibelix(name, str(tmp_path / name))
        obj = json.load(open(tmp_path / name / "config.json"))
        arch = resolve_architecture(obj)
        man = plan_manifest(arch.build_plan(arch.config_class.from_dict(obj)))
        with safe_open(str(tmp_path / name / "model.safetensors"), framework="pt") as f:
            found = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
        check_manifest(man, found)
        assert set(found) == {s.name for s in man}
    assert "mixed" in ROUTED and "only_dense" not in ROUTED


# -- the plain implementation's mechanisms, by hand ------------------------------------------------------------------

def test_plain_tanh_norm_and_soft_cap():
    w = {"n": torch.tensor([2.0, -1.0], dtype=P.F), "n.b": torch.tensor([0.5, 0.25], dtype=P.F),
         "n.alpha": torch.tensor(0.5, dtype=P.F)}
    x = torch.tensor([[2.0, -4.0]], dtype=P.F)
    got = P.tanh_norm(x, w, "n")
    assert torch.allclose(got, torch.tensor([[2 * math.tanh(1.0) + 0.5, math.tanh(2.0) + 0.25]], dtype=P.F))
    assert abs(float(P.soft_cap(torch.tensor(1000.0, dtype=P.F), 30.0)) - 30.0) < 1e-9
    assert abs(float(P.soft_cap(torch.tensor(0.3, dtype=P.F), 30.0)) - 30 * math.tanh(0.01)) < 1e-12


def test_plain_rotation_pairs_and_leaves_the_rest():
    x = torch.arange(1.0, 7.0, dtype=P.F).view(1, 1, 6).repeat(3, 1, 1)          # 3 positions, dims 4 of 6
    out = P.rotate_half_split(x, 4, 100.0)
    assert torch.equal(out[0], x[0]) and torch.equal(out[:, :, 4:], x[:, :, 4:])
    for p in (1, 2):
        for i, f in enumerate((1.0, 100.0 ** -0.5)):
            u, v = 1.0 + i, 3.0 + i
            assert abs(float(out[p, 0, i]) - (u * math.cos(p * f) - v * math.sin(p * f))) < 1e-12
            assert abs(float(out[p, 0, i + 2]) - (v * math.cos(p * f) + u * math.sin(p * f))) < 1e-12


def test_plain_window_sees_itself_and_the_tokens_before():
    T = 6
    q = torch.zeros(T, 2, dtype=P.F)
    k = torch.zeros(T, 2, dtype=P.F)
    v = torch.arange(T, dtype=P.F).view(T, 1)
    out = P.windowed_softmax_attention(q, k, v, 1.0, 3)                         # equal scores: the mean of what is seen
    assert torch.allclose(out[:, 0], torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=P.F))
    assert torch.allclose(P.windowed_softmax_attention(q, k, v, 1.0, 1)[:, 0], v[:, 0])


def test_plain_lightning_is_the_sum_it_says_and_carries_its_state():
    g = torch.Generator().manual_seed(1)
    W, H, d, dv, T = 10, 2, 3, 4, 7
    w = {k: torch.randn(s, generator=g, dtype=P.F) for k, s in
         (("m.q", (H * d, W)), ("m.k", (H * d, W)), ("m.v", (H * dv, W)), ("m.g", (H * dv, W)), ("m.o", (W, H * dv)))}
    w["m.norm"] = torch.rand(H * dv, generator=g, dtype=P.F) + 0.5
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 1.0]}
    h = torch.randn(T, W, generator=g, dtype=P.F)
    y, S = P.lightning_attention(h, w, "m.", m, 1e-5)
    # by the closed form: o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s, all heads normed together
    q, k, v = (P.silu(h @ w["m." + n].T) for n in ("q", "k", "v"))
    o = torch.zeros(T, H * dv, dtype=P.F)
    for t in range(T):
        for hd in range(H):
            for s in range(t + 1):
                o[t, hd * dv:(hd + 1) * dv] += m["decay"][hd] ** (t - s) * \
                    (q[t, hd * d:(hd + 1) * d] @ k[s, hd * d:(hd + 1) * d]) * v[s, hd * dv:(hd + 1) * dv]
    want = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * w["m.norm"] * torch.sigmoid(h @ w["m.g"].T)) @ w["m.o"].T
    assert torch.allclose(y, want, atol=1e-10)
    y1, S1 = P.lightning_attention(h[:4], w, "m.", m, 1e-5)
    y2, S2 = P.lightning_attention(h[4:], w, "m.", m, 1e-5, state=S1)
    assert torch.allclose(torch.cat([y1, y2]), y, atol=1e-10) and torch.allclose(S2, S, atol=1e-12)


def test_plain_router_groups_corrections_and_identity():
    # 6 outputs in 3 groups of 2, 1 group kept, 2 picks; equal logits: every score is 1/6
    w = {"r.router": torch.zeros(6, 2, dtype=P.F),
         "r.correction": torch.tensor([-0.9, -0.8, -0.5, -0.7, -0.95, -0.6], dtype=P.F)}
    r = {"experts": 4, "identity": 2, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    picks = P.route(torch.ones(1, 2, dtype=P.F), w, "r.", r)[0]
    # every choice score is negative; group 1 holds the largest (-0.5 + 1/6); both of its outputs are picked, in order,
    # though output 5 of group 2 has a larger choice score than output 3; the weight is the score without correction
    assert [e for e, _ in picks] == [2, 3] and all(abs(wt - 0.5) < 1e-12 for _, wt in picks)
    r["groups"] = {"count": 3, "keep": 2}
    assert [e for e, _ in P.route(torch.ones(1, 2, dtype=P.F), w, "r.", r)[0]] == [2, 5]
    # an identity pick gives the input back, times its weight; no shared expert
    mlp = {"router": {"experts": 0, "identity": 2, "top": 1, "scale": 2.0, "groups": {"count": 1, "keep": 1}}}
    w2 = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 0.0]], dtype=P.F), "r.correction": torch.zeros(2, dtype=P.F)}
    h = torch.tensor([[2.0, 5.0]], dtype=P.F)
    s0 = math.exp(2.0) / (math.exp(2.0) + 1.0)
    assert torch.allclose(P.mixture_of_experts(h, w2, "r.", mlp), 2.0 * s0 * h)


def test_plain_differential_attention_by_hand():
    """One head, one key/value head, no rotation, window 2: both maps by hand."""
    g = torch.Generator().manual_seed(3)
    W, d, dv, T = 5, 2, 3, 4
    w = {"a." + n: torch.randn(s, generator=g, dtype=P.F) for n, s in
         (("q", (2 * d, W)), ("k", (2 * d, W)), ("v", (dv, W)), ("g", (1, W)), ("o", (W, dv)))}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        w["a." + n] = torch.randn(d, generator=g, dtype=P.F) * 0.5
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 0.4, "diff": 0.2, "mask": {"size": 2}}
    h = torch.randn(T, W, generator=g, dtype=P.F)
    got = P.differential_attention(h, w, "a.", m, 1e-5)
    q, k, v = h @ w["a.q"].T, h @ w["a.k"].T, h @ w["a.v"].T
    lam = math.exp(float(w["a.lq1"] @ w["a.lk1"])) - math.exp(float(w["a.lq2"] @ w["a.lk2"])) + 0.2
    rows = []
    for t in range(T):
        maps = []
        for mp in range(2):
            js = [j for j in (t - 1, t) if j >= 0]
            sc = torch.tensor([float(q[t, mp * d:(mp + 1) * d] @ k[j, mp * d:(mp + 1) * d]) * 0.4 for j in js], dtype=P.F)
            p = torch.softmax(sc, 0)
            maps.append(sum(p[i] * v[j] for i, j in enumerate(js)))
        o = maps[0] - lam * maps[1]
        o = o / torch.sqrt((o * o).mean() + 1e-5) * 0.8 * torch.sigmoid(h[t] @ w["a.g"][0])
        rows.append(o @ w["a.o"].T)
    assert torch.allclose(got, torch.stack(rows), atol=1e-10)
