"""Small Potodra configurations for the tests, different in every size and option, with random weights."""
from __future__ import annotations

import os

import torch
from safetensors import safe_open

from exl3_server_b200 import write_random_model
from exl3_server_b200.config.potodra import PotodraConfig, PotodraLayer
from exl3_server_b200.weights.safetensors_io import write_safetensors


def attn(heads, kv_heads, dim, vdim, scale, window=None, keep=0, softcap=None, base=10000.0, dims=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    if dims != 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
    return m


def mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def par(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, groups=(1, 1), shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
           "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def L(kind, mixer, mlp):
    return PotodraLayer(kind, mixer, mlp)


def cfg(vocab, width, streams, eps, scale, layers):
    return PotodraConfig(vocab=vocab, width=width, streams=streams, norm_eps=eps, embedding_scale=scale, layers=layers)


CONFIGS = {
    # every kind of layer with both feed-forwards; two streams; windows of 50 and 33 positions (no multiple of a page)
    # that keep 5 and 70 first keys (more than a page); part of a head rotated; values narrower and wider than keys;
    # three value heads on one query/key head in the delta rule and one on one; three and two taps; groups of three
    # experts of which two groups of three are kept, one group, no shared expert; a layer without a feed-forward
    "mixed": cfg(211, 96, 2, 1e-5, 2.5, [
        L("attention", attn(4, 2, 24, 16, 0.21, window=50, keep=5, softcap=9.0, dims=12), dense(160)),
        L("mlstm", mlstm(3, 16, 24, 8.0), moe(40, 1.2, 9, 2, groups=(3, 2), shared=(56, 2.0))),
        L("parallel", par(attn(6, 3, 16, 40, 0.3, base=500.0, dims=8), delta(3, 1, 16, 8, 3), 0.7, 0.4), moe(48, 2.5, 5, 3)),
        L("attention", attn(2, 2, 32, 24, 0.18, window=33, keep=70, softcap=30.0), None),
        L("parallel", par(attn(2, 1, 8, 8, 0.35), delta(2, 2, 24, 16, 2), -0.5, 1.1), dense(72)),
        L("mlstm", mlstm(1, 8, 40, 20.0), dense(56)),
    ]),
    # sizes that are multiples of nothing, one stream (the arrangement is then an ordinary pre-norm residual), a
    # window of 7 positions that keeps one first key, a window that keeps none, no soft cap, no rotation, one tap
    # (no convolution state), five taps, one expert, every expert picked, an embedding scale of one
    "odd": cfg(97, 100, 1, 1e-6, 1.0, [
        L("attention", attn(3, 3, 10, 6, 0.4, window=7, keep=1, dims=0), moe(12, 0.8, 1, 1, shared=(20, 0.5))),
        L("parallel", par(attn(1, 1, 12, 20, 0.25, dims=6), delta(1, 1, 12, 20, 1), 1.0, 1.0), dense(30)),
        L("mlstm", mlstm(2, 12, 20, 3.0), moe(16, 4.0, 4, 4, groups=(2, 2))),
        L("attention", attn(2, 1, 14, 14, 0.3, window=20, keep=0, softcap=5.0, dims=14), dense(44)),
        L("parallel", par(attn(4, 2, 6, 10, 0.5, base=77.0), delta(4, 2, 20, 12, 5), 0.3, -0.8), None),
    ]),
    # four streams, heads of 64 and 128 features (the sizes of the tensor-core attention kernels) in the plain causal
    # attention, keys of 64 and 128 in the recurrences, a window of three pages that keeps one page exactly
    "wide": cfg(301, 128, 4, 1e-5, 4.0, [
        L("parallel", par(attn(4, 2, 64, 64, 0.11), delta(2, 1, 64, 64, 4), 0.5, 0.5), dense(192)),
        L("attention", attn(4, 1, 64, 64, 0.12, window=192, keep=64, softcap=15.0), moe(64, 1.75, 8, 2, groups=(4, 2), shared=(64, 1.25))),
        L("mlstm", mlstm(2, 128, 64, 12.0), dense(128)),
        L("parallel", par(attn(2, 2, 128, 128, 0.08, dims=64), delta(2, 2, 128, 32, 4), 0.9, 0.2), None),
        L("mlstm", mlstm(2, 64, 128, 14.0), None),
    ]),
    # each mechanism alone
    "only_attention": cfg(128, 64, 4, 1e-5, 2.0, [L("attention", attn(4, 2, 32, 16, 0.25, window=70, keep=9, softcap=12.0, dims=16), None)]),
    "only_full_attention": cfg(128, 64, 2, 1e-5, 2.0, [L("parallel", par(attn(4, 2, 16, 24, 0.3, dims=8), delta(1, 1, 8, 8, 2), 1.0, 0.0), None)]),
    "only_mlstm": cfg(128, 64, 2, 1e-5, 2.0, [L("mlstm", mlstm(2, 16, 24, 10.0), None)]),
    "only_delta": cfg(128, 64, 2, 1e-5, 2.0, [L("parallel", par(attn(1, 1, 8, 8, 0.3), delta(4, 2, 16, 24, 4), 0.0, 1.0), None)]),
    "only_moe": cfg(128, 64, 1, 1e-5, 1.5, [L("mlstm", mlstm(1, 8, 8, 10.0), moe(24, 1.0, 12, 3, groups=(4, 2), shared=(16, 3.0)))]),
    "only_dense": cfg(128, 64, 5, 1e-5, 1.5, [L("mlstm", mlstm(1, 8, 8, 10.0), dense(80))]),
}


def random_config(seed: int) -> PotodraConfig:
    """A configuration drawn from a seed: two to five layers of any kind in any order, every size, count and constant
    drawn anew (within what the design allows), a dense, routed or no feed-forward beside each."""
    import random
    r = random.Random(seed)
    width = r.choice([48, 72, 80, 104, 136])

    def an_attention(windowed: bool):
        kv = r.randint(1, 3)
        dim = r.choice([6, 8, 16, 24, 32, 64])
        window = r.choice([1, 2, 5, 31, 64, 65, 200]) if windowed and r.random() < 0.8 else None
        return attn(kv * r.randint(1, 4), kv, dim, r.choice([8, 12, 16, 32, 64]), r.uniform(0.1, 0.3), window=window,
                    keep=r.choice([0, 1, 3, 64, 100]) if window else 0,
                    softcap=r.choice([None, 5.0, 25.0, 50.0]) if windowed else None,
                    base=r.choice([100.0, 10000.0, 1e6]), dims=r.choice([0, 2, dim // 2 * 2, dim]))

    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["attention", "mlstm", "parallel"])
        if kind == "attention":
            mixer = an_attention(True)
        elif kind == "mlstm":
            mixer = mlstm(r.randint(1, 4), r.choice([4, 8, 12, 16, 32, 40]), r.choice([6, 8, 16, 24, 32]),
                          r.choice([2.0, 10.0, 12.0, 30.0]))
        else:
            g = r.randint(1, 2)
            mixer = par(an_attention(False), delta(g * r.randint(1, 3), g, r.choice([4, 8, 12, 16, 32]),
                                                   r.choice([6, 8, 16, 24]), r.randint(1, 5)),
                        r.uniform(0.2, 1.2), r.uniform(0.2, 1.2))
        what = r.random()
        if what < 0.25:
            mlp = None
        elif what < 0.5:
            mlp = dense(r.choice([24, 40, 100]))
        else:
            per, groups = r.randint(1, 4), r.randint(1, 4)
            keep = r.randint(1, groups)
            mlp = moe(r.choice([8, 24, 40]), r.choice([0.7, 1.3, 7.0]), per * groups, r.randint(1, keep * per),
                      groups=(groups, keep), shared=r.choice([None, (16, 1.0), (40, 3.0)]))
        layers.append(L(kind, mixer, mlp))
    return cfg(r.randint(40, 300), width, r.randint(1, 5), r.choice([1e-6, 1e-5, 1e-4]), r.uniform(0.5, 4.0), layers)


RANDOM_SEEDS = list(range(200, 210))
CONFIGS.update({f"random{seed}": random_config(seed) for seed in RANDOM_SEEDS})

ROUTED = {name for name, c in CONFIGS.items() if any(l.mlp and l.mlp["kind"] == "moe" for l in c.layers)}


def make_potodra(name: str, folder: str, std: float = 0.06) -> str:
    """std 0.06: scores of order one, so that a wrong key, position or slot shows far above rounding (a little below the
    other designs' 0.08: squares, bounded gates and exponentials of gate sums multiply bfloat16 rounding layer by layer).  What random
    weights of that size would hide or make meaningless is drawn otherwise: the streams' mixing matrices near the
    identity with off-diagonal entries of a few tenths, read weights spread around one, write weights of both signs,
    sinks of -1 .. 2 (a sink left out changes every row), larger routers and corrections of both signs (some choice
    scores negative), gate biases that let the forget gate stand near one and the input gate vary, decays spread over
    0.3 .. 0.999 per step, taps of order one, larger low-rank pairs."""
    write_random_model(CONFIGS[name], folder, seed=2203 + sum(map(ord, name)), std=std, norm_std=0.1,
                       dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    with safe_open(path, framework="pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    g = torch.Generator().manual_seed(11)
    rnd = lambda shape: torch.rand(shape, generator=g)
    for k in sorted(tensors):
        t = tensors[k]
        last = k.rsplit(".", 1)[-1]
        if ".hc" in k and last == "mix":
            tensors[k] = (torch.eye(t.shape[0]) * (0.7 + 0.4 * rnd(())) + (rnd(t.shape) - 0.5) * 0.6).to(torch.bfloat16)
        elif ".hc" in k and last in ("in", "out"):
            # read weights of one sign (a read in which the streams nearly cancel would multiply every rounding error
            # before it); write weights of both signs
            v = 0.4 + 0.9 * rnd(t.shape)
            if t.numel() > 1 and last == "out":
                v[-1] = -v[-1] * 0.5
            tensors[k] = v.to(torch.bfloat16)
        elif last == "sink":
            tensors[k] = (3.0 * rnd(t.shape) - 1.0).to(torch.bfloat16)
        elif k.endswith(".mlp.router"):
            tensors[k] = (t.float() * 3.0).to(torch.bfloat16)
        elif k.endswith(".mlp.correction"):
            tensors[k] = ((rnd(t.shape) - 0.7) * 0.6).to(torch.bfloat16)
        elif k.endswith(".conv"):
            tensors[k] = ((rnd(t.shape) - 0.4) * 1.5).to(torch.bfloat16)
        elif last == "A_log":
            tensors[k] = (torch.log(0.05 + 1.5 * rnd(t.shape))).to(torch.bfloat16)
        elif last == "dt_bias":
            tensors[k] = (2.0 * rnd(t.shape) - 2.0).to(torch.bfloat16)
        elif last in ("a1", "a2", "g1", "g2") or k.endswith(".mix.right.b") or k.endswith(".mix.i") or k.endswith(".mix.f"):
            tensors[k] = (t.float() * 2.0).to(torch.bfloat16)
        elif k.endswith(".f.b"):
            tensors[k] = (1.0 + 3.0 * rnd(t.shape)).to(torch.bfloat16)
        elif k.endswith(".i.b"):
            tensors[k] = (rnd(t.shape) - 0.5).to(torch.bfloat16)
        elif last == "b" and (k.endswith(".q.b") or k.endswith(".k.b") or k.endswith(".v.b")):
            tensors[k] = ((rnd(t.shape) - 0.5) * 0.6).to(torch.bfloat16)
    write_safetensors(path, tensors.items(), metadata={"format": "pt"})
    return folder
