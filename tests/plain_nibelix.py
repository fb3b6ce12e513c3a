"""A plain, slow implementation of the Nibelix decoder: whole sequences, no cache, no state carried between calls,
float64, one function per mechanism.  It shares no code with the package: config.json is read with ``json``, the
weights with the ``safetensors`` library, and everything is plain torch arithmetic on the CPU.  Attention builds the
full score matrix with its mask; the recurrence is a Python loop over tokens; the router is a loop over tokens.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Tuple

import torch
from safetensors import safe_open

F = torch.float64


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F)
    return out


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def tanh_norm(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """The layers' norm: no statistics at all, ``tanh(alpha x) * weight + bias`` with one learned scalar alpha."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def rotate_half_split(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, n, d] at positions 0 .. T-1: feature i of the first ``dims`` is paired with feature i + dims/2; the
    rest stay as they are."""
    if dims == 0:
        return x
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    a = torch.arange(x.shape[0], dtype=F)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    return out


def windowed_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """q [T, d], k [T, d], v [T, dv] of one head: query i sees keys j with 0 <= i - j < window."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < window)
    s = s.masked_fill(~seen, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                           probe: Optional[dict] = None) -> torch.Tensor:
    """Two softmax attention maps per head over the same values, the second subtracted from the first."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff = m["diff"]
    q = (h @ w[p + "q"].T).view(T, H * 2, d)                     # head by head: [map 1, map 2]
    k = (h @ w[p + "k"].T).view(T, G * 2, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    if m.get("rot") is not None:
        q = rotate_half_split(q, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_half_split(k, m["rot"]["dims"], m["rot"]["base"])
    window = m["mask"]["size"] if m.get("mask") is not None else T      # no mask in the configuration: every key before
    lam = math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        a1 = windowed_softmax_attention(q[:, 2 * hd], k[:, 2 * g], v[:, g], m["scale"], window)
        a2 = windowed_softmax_attention(q[:, 2 * hd + 1], k[:, 2 * g + 1], v[:, g], m["scale"], window)
        o = unit_rms(a1 - lam * a2, eps) * (1.0 - diff)
        outs.append(o * gate[:, hd:hd + 1])
    if probe is not None:
        probe["q"], probe["k"], probe["lambda"] = q, k, lam
    return torch.cat(outs, dim=-1) @ w[p + "o"].T


def lightning_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                        state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """A matrix state per head with one fixed decay; returns the mixer's output and the state after the last token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F) if state is None else state.clone()
    decay = torch.tensor(m["decay"], dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    y = unit_rms(o.reshape(T, H * dv), eps) * w[p + "norm"]       # all heads normed together
    y = y * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, S


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def small_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, r: dict,
          margins: Optional[list] = None) -> List[List[Tuple[int, float]]]:
    """Per token the chosen experts and their weights.  Router outputs number ``experts + identity``; the choice is
    by score plus correction among the experts of the best groups, the weight is the score alone times a constant.
    ``margins`` gets, per token, how close the choice was: the smallest gap between something chosen and something
    left out (groups and experts)."""
    n = r["experts"] + r["identity"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    per = n // r["groups"]["count"]
    out = []
    for t in range(h.shape[0]):
        c = choice[t]
        by_group = sorted(range(r["groups"]["count"]), key=lambda g: -float(c[g * per:(g + 1) * per].max()))
        best = by_group[:r["groups"]["keep"]]
        open_ = sorted((e for e in range(n) if e // per in best), key=lambda e: -float(c[e]))
        chosen = open_[:r["top"]]
        if margins is not None:
            gap = float("inf")
            if len(by_group) > len(best):
                gap = float(c[best[-1] * per:(best[-1] + 1) * per].max() - c[by_group[len(best)] * per:(by_group[len(best)] + 1) * per].max())
            if len(open_) > len(chosen):
                gap = min(gap, float(c[chosen[-1]] - c[open_[len(chosen)]]))
            margins.append(gap)
        out.append([(e, float(s[t, e]) * r["scale"]) for e in chosen])
    return out


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
                       margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    y = torch.zeros_like(h)
    for t, picks in enumerate(route(h, w, p, r, margins)):
        for e, weight in picks:
            if e >= r["experts"]:                                 # an identity expert: the input itself
                y[t] += weight * h[t]
            else:
                y[t] += weight * small_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        y = y + small_expert(h, w, p + "shared.") * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return y


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h1 = tanh_norm(x, w, p + "norm1")
        if layer["type"] == "lightning":
            y, _ = lightning_attention(h1, w, p + "mix.", layer["mixer"], eps)
        else:
            y = differential_attention(h1, w, p + "mix.", layer["mixer"], eps)
        total = y * w[p + "ls1"]
        if layer.get("mlp") is not None:
            h2 = tanh_norm(x, w, p + "norm2")
            if layer["mlp"]["kind"] == "dense":
                f = dense_feed_forward(h2, w, p + "mlp.")
            else:
                f = mixture_of_experts(h2, w, p + "mlp.", layer["mlp"], margins)
            total = total + f * w[p + "ls2"]
        x = x + m * total
        if layers_out is not None:
            layers_out.append(x.clone())
    z = tanh_norm(x, w, "final.norm") @ w["head"].T
    return soft_cap(z, cfg["logit_softcap"]) if cfg.get("logit_softcap") else z


class PlainNibelix:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_weights(model_dir)

        self._memo: dict = {}

    def run(self, tokens: List[int]) -> Tuple[torch.Tensor, float]:
        """(logits, the smallest margin of any router's choice over the sequence; infinite without routers)."""
        key = tuple(tokens)
        if key not in self._memo:
            margins: list = []
            self._memo[key] = (forward(self.cfg, self.w, tokens, None, margins), min(margins, default=float("inf")))
        return self._memo[key]

    def logits(self, tokens: List[int]) -> torch.Tensor:
        return self.run(tokens)[0]

    def closest_call(self, tokens: List[int]) -> float:
        """The smallest margin of any router's choice over the sequence (infinite without routers)."""
        return self.run(tokens)[1]

    def layers(self, tokens: List[int]) -> torch.Tensor:
        out: list = []
        forward(self.cfg, self.w, tokens, out)
        return torch.stack(out)

    def greedy(self, prompt: List[int], n: int) -> List[int]:
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(torch.argmax(forward(self.cfg, self.w, toks)[-1])))
        return toks[len(prompt):]
