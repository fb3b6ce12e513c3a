"""Small Nibelix configurations for the tests, different in every size and option, with random weights."""
from __future__ import annotations

import math
import os

import torch
from safetensors import safe_open

from exl3_server_b200 import write_random_model
from exl3_server_b200.config.nibelix import NibelixConfig, NibelixLayer
from exl3_server_b200.weights.safetensors_io import write_safetensors


def light(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def attn(heads, kv_heads, dim, vdim, scale, diff, window=None, base=10000.0, dims=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window:
        m["mask"] = {"size": window}
    if dims != 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, scale, groups=(1, 1), shared=None):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": identity, "top": top, "scale": scale,
                      "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def L(kind, mixer, mlp):
    return NibelixLayer(kind, mixer, mlp)


CONFIGS = {
    # every kind of layer and feed-forward in both pairings; two and three kv heads; keys narrower and wider than
    # values, two maps that are not as wide as the values together; part of a map rotated; windows of 50 and 33
    # positions (no multiple of a page) and a layer without a window; groups of which two of three are kept, one
    # group, no identity outputs and three; one, two and three picks; no shared expert; a layer without a feed-forward;
    # a dense feed-forward beside attention; states that are not square
    "mixed": NibelixConfig(vocab=211, width=96, norm_eps=1e-5, residual_mult=0.7, logit_softcap=12.0, layers=[
        L("attention", attn(4, 2, 24, 16, 0.21, 0.25, window=50, dims=12), dense(160)),
        L("lightning", light(3, 16, 24, (0.7, 0.97, 0.999)), moe(40, 9, 0, 2, 1.5, groups=(3, 2), shared=56)),
        L("attention", attn(6, 3, 16, 40, 0.3, 0.4, base=500.0, dims=8), moe(48, 5, 3, 3, 0.8, groups=(2, 2))),
        L("lightning", light(2, 32, 16, (0.9, 0.995)), None),
        L("attention", attn(2, 2, 32, 24, 0.18, 0.15, window=33), moe(32, 6, 2, 1, 2.5, groups=(4, 1), shared=24)),
        L("lightning", light(4, 8, 8, (0.5, 0.8, 0.95, 0.99)), dense(72)),
    ]),
    # sizes that are multiples of nothing: maps of 10 features, values of 6, a width of 100, a state of 12 x 20, a
    # window of 7 positions, one query head a kv head, a decay of exactly one, all of a map rotated, no rotation,
    # a router whose outputs are all identity but one, no soft cap
    "odd": NibelixConfig(vocab=77, width=100, norm_eps=2e-6, residual_mult=0.5, logit_softcap=0.0, layers=[
        L("attention", attn(3, 3, 10, 6, 0.3, 0.2, window=7, base=300.0), moe(30, 1, 3, 2, 1.0)),
        L("lightning", light(2, 12, 20, (1.0, 0.9)), dense(70)),
        L("attention", attn(5, 1, 6, 12, 0.35, 0.5, dims=0), None),
        L("lightning", light(1, 20, 12, (0.98,)), moe(22, 7, 0, 7, 1.0, shared=10)),
    ]),
    # maps of 64 features (a key row of 128) and values of 128, states of 64 x 128 and 128 x 64, a window of exactly
    # two pages, eight query heads on a kv head, long decays, sixteen router outputs in four groups
    "wide": NibelixConfig(vocab=300, width=128, norm_eps=1e-6, residual_mult=1.0, logit_softcap=30.0, layers=[
        L("lightning", light(2, 64, 128, (0.95, 0.998)), dense(320)),
        L("attention", attn(8, 1, 64, 128, 0.125, 0.3, window=128, base=250000.0, dims=32),
          moe(64, 14, 2, 4, 2.0, groups=(4, 2), shared=96)),
        L("lightning", light(2, 128, 64, (0.99, 0.9)), moe(96, 8, 0, 2, 1.0, groups=(2, 1))),
        L("attention", attn(4, 2, 32, 64, 0.18, 0.1, window=100), dense(192)),
    ]),
    # key rows of 64 features, the tensor-core attention kernels' other shape: values narrower than the row (padded), a
    # window shorter than a page, one kv head for 4 and for 12 query heads (24 maps on a kv head: more than the decode
    # kernel takes, so decoding falls to the CUDA-core kernel while prompts stay on the tensor cores), no window
    "tensor": NibelixConfig(vocab=160, width=128, norm_eps=1e-6, residual_mult=0.6, logit_softcap=15.0, layers=[
        L("attention", attn(4, 1, 32, 48, 0.18, 0.3, window=20), dense(96)),
        L("attention", attn(12, 1, 32, 64, 0.18, 0.2, dims=16), moe(24, 4, 1, 2, 1.2, shared=32)),
    ]),
    # one mechanism alone (the smallest feed-forward there can be where the mechanism is a mixer)
    "only_attention": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("attention", attn(4, 2, 32, 24, 0.18, 0.3, window=70, dims=16), None)]),
    "only_attention_64": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("attention", attn(4, 2, 64, 64, 0.09, 0.3, window=70, dims=32), None)]),
    "only_full_attention": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("attention", attn(4, 1, 16, 48, 0.25, 0.6, dims=8), None)]),
    "only_lightning": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("lightning", light(4, 24, 40, (0.6, 0.9, 0.99, 0.9995)), None)]),
    "only_dense": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("lightning", light(1, 8, 8, (0.5,)), dense(200))]),
    "only_routed": NibelixConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, logit_softcap=20.0, layers=[
        L("lightning", light(1, 8, 8, (0.5,)), moe(48, 10, 2, 3, 1.7, groups=(3, 2), shared=40))]),
}

def random_config(seed: int) -> NibelixConfig:
    """A configuration drawn from a seed: two to five layers of either kind in any order, every size, count and constant
    drawn anew (within what the design allows), a dense, routed or no feed-forward beside each."""
    import random
    r = random.Random(seed)
    width = r.choice([48, 72, 80, 104, 136])
    layers = []
    for _ in range(r.randint(2, 5)):
        if r.random() < 0.5:
            heads = r.randint(1, 4)
            mixer = light(heads, r.choice([4, 8, 12, 16, 32, 40]), r.choice([6, 8, 16, 24, 32]),
                          [r.choice([1.0, 0.999, 0.97, 0.9, 0.6, 0.3]) for _ in range(heads)])
            kind = "lightning"
        else:
            kv = r.randint(1, 3)
            dim = r.choice([6, 8, 16, 24, 32, 64])
            mixer = attn(kv * r.randint(1, 4), kv, dim, r.choice([8, 12, 16, 32, 64, 128]), r.uniform(0.1, 0.3),
                         r.uniform(0.05, 0.7), window=r.choice([None, 1, 2, 5, 31, 64, 65, 200]),
                         base=r.choice([100.0, 10000.0, 1e6]), dims=r.choice([0, 2, dim // 2 * 2, dim]))
            kind = "attention"
        what = r.random()
        if what < 0.25:
            mlp = None
        elif what < 0.5:
            mlp = dense(r.choice([24, 40, 100]))
        else:
            per, groups = r.randint(1, 4), r.randint(1, 4)
            n = per * groups
            identity = r.randint(0, min(2, n - 1)) if n > 1 else 0
            keep = r.randint(1, groups)
            mlp = moe(r.choice([8, 24, 40]), n - identity, identity, r.randint(1, keep * per), r.uniform(0.5, 2.5),
                      groups=(groups, keep), shared=r.choice([None, 16, 40]))
        layers.append(L(kind, mixer, mlp))
    return NibelixConfig(vocab=r.randint(40, 300), width=width, norm_eps=r.choice([1e-6, 1e-5, 1e-4]),
                         residual_mult=r.uniform(0.3, 1.0), logit_softcap=r.choice([0.0, 10.0, 30.0, 50.0]), layers=layers)


RANDOM_SEEDS = list(range(100, 112))
CONFIGS.update({f"random{seed}": random_config(seed) for seed in RANDOM_SEEDS})

ROUTED = {name for name, c in CONFIGS.items() if any(l.mlp and l.mlp["kind"] == "moe" for l in c.layers)}


def make_nibelix(name: str, folder: str, std: float = 0.08) -> str:
    """std 0.08: scores of order one, so that a wrong key, position or slot shows far above rounding.  What random
    weights of that size would hide is made larger: the four vectors behind an attention layer's lambda (so that
    lambda is not just the configuration's constant, nor near 1), the routers' matrices and corrections (so that the
    correction changes the choice and some choice scores are negative), the norms' biases, and the layer scales are
    spread over 0.5 .. 1.5."""
    write_random_model(CONFIGS[name], folder, seed=1511 + sum(map(ord, name)), std=std, norm_std=0.1,
                       dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    with safe_open(path, framework="pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    g = torch.Generator().manual_seed(7)
    for k in sorted(tensors):
        t = tensors[k]
        if k.rsplit(".", 1)[-1] in ("lq1", "lq2"):
            # lq1 . lk1 = log of 0.6 .. 0.8 and lq2 . lk2 = log of 1.1 .. 1.4: lambda is the constant less 0.3 .. 0.8,
            # well away from 1, where the two maps would cancel and the norm after them blow rounding up
            which = k[-1]
            lo, span = (0.6, 0.2) if which == "1" else (1.1, 0.3)
            target = math.log(lo + span * float(torch.rand((), generator=g)))
            lq = torch.rand(t.shape, generator=g) - 0.5
            lk = torch.rand(t.shape, generator=g) + 0.25
            lk = lk * target / float((lq.to(torch.bfloat16).float() * lk).sum())
            tensors[k] = lq.to(torch.bfloat16)
            tensors[k[:-2] + "k" + which] = lk.to(torch.bfloat16)
        elif k.rsplit(".", 1)[-1] in ("lk1", "lk2"):
            continue
        elif k.endswith(".mlp.router"):
            tensors[k] = (t.float() * 3.0).to(torch.bfloat16)
        elif k.endswith(".mlp.correction"):
            tensors[k] = ((torch.rand(t.shape, generator=g) - 0.7) * 0.3).to(torch.bfloat16)
        elif k.endswith(".ls1") or k.endswith(".ls2"):
            tensors[k] = (0.5 + torch.rand(t.shape, generator=g)).to(torch.bfloat16)
        elif k.endswith(".alpha"):
            tensors[k] = (0.6 + 0.8 * torch.rand((), generator=g)).to(torch.bfloat16)
    write_safetensors(path, tensors.items(), metadata={"format": "pt"})
    return folder
