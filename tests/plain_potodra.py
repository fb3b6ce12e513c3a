"""A plain, slow implementation of the Potodra decoder: whole sequences, no cache, no state carried between calls,
float64, one function per mechanism.  It shares no code with the package: config.json is read with ``json``, the
weights with the ``safetensors`` library, and everything is plain torch arithmetic on the CPU.  Attention builds the
full score matrix with its mask; the recurrences and the short convolutions are Python loops over tokens; the router is
a loop over tokens.
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


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(x, torch.zeros_like(x))


def log_sigmoid(x: torch.Tensor) -> torch.Tensor:
    return -softplus(-x)


def rotate(x: torch.Tensor, dims: int, base: float, layout: str) -> torch.Tensor:
    """x [T, n, d] at positions 0 .. T-1.  Of the first ``dims`` features, ``half``: feature i goes with feature
    i + dims/2; ``interleaved``: feature 2i with 2i + 1.  The rest stay as they are."""
    if dims == 0:
        return x
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    a = torch.arange(x.shape[0], dtype=F)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return out


def visible(T: int, window: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (i - j < window or j < keep_first); window 0: no window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, layout: str,
                      scores_out: Optional[list] = None) -> torch.Tensor:
    """Grouped-query attention with biases on q, k, v; optional in ``m``: ``rot``, ``softcap``, ``mask`` (a window that
    keeps the first tokens too), and a learned sink per head (the tensor ``sink``) in the softmax's denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    if m.get("rot"):
        q = rotate(q, m["rot"]["dims"], m["rot"]["base"], layout)
        k = rotate(k, m["rot"]["dims"], m["rot"]["base"], layout)
    mask = m.get("mask") or {}
    ok = visible(T, int(mask.get("size", 0)), int(mask.get("keep_first", 0)))
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        if scores_out is not None:
            scores_out.append(s.clone())
        s = s.masked_fill(~ok, -math.inf)
        e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        den = e.sum(dim=-1, keepdim=True)
        if p + "sink" in w:
            den = den + torch.exp(w[p + "sink"][hd] - s.max(dim=-1, keepdim=True).values)
        outs.append((e / den) @ v[:, g])
    return torch.cat(outs, dim=-1) @ w[p + "o"].T


def mlstm(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """A matrix memory per head with exponential gates kept in range by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F)
        n = torch.zeros(d, dtype=F)
        mx = torch.zeros((), dtype=F)
        for t in range(T):
            m_new = torch.maximum(gf[t, hd] + mx, gi[t, hd])
            a, b = torch.exp(gf[t, hd] + mx - m_new), torch.exp(gi[t, hd] - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            den = torch.maximum(torch.abs(n @ q[t, hd]), torch.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, n - 1 - j] x[t - j, c], zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(n):
            if t - j >= 0:
                y[t] += taps[:, n - 1 - j] * x[t - j]
    return y


def gated_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """The gated delta rule: a matrix state per head that decays per key channel, is corrected towards the token's
    value along the token's key, and is read after the write."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    dt = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, d)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    o = unit_rms(out, eps) * w[p + "norm"]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = softmax_attention(h, w, p + "left.", m["left"], "interleaved")
    right = gated_delta(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def clamped_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z: torch.Tensor, correction: torch.Tensor, groups: int, keep: int, top: int) -> Tuple[List[int], float]:
    """One token's picks from its router logits, and the margin of the closest decision."""
    s = torch.sigmoid(z)
    c = s + correction
    n = c.numel()
    size = n // groups
    gs = torch.stack([torch.topk(c[g * size:(g + 1) * size], min(2, size)).values.sum() for g in range(groups)])
    order = sorted(range(groups), key=lambda g: (-float(gs[g]), g))
    kept = order[:keep]
    margin = float(gs[order[keep - 1]] - gs[order[keep]]) if keep < groups else float("inf")
    allowed = [e for e in range(n) if e // size in kept]
    ranked = sorted(allowed, key=lambda e: (-float(c[e]), e))
    if top < len(ranked):
        margin = min(margin, float(c[ranked[top - 1]] - c[ranked[top]]))
    return ranked[:top], margin


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
                       margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    z = h @ w[p + "router"].T
    s = torch.sigmoid(z)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        picks, margin = route(z[t], w[p + "correction"], r["groups"]["count"], r["groups"]["keep"], r["top"])
        if margins is not None:
            margins.append(margin)
        for e in picks:
            out[t] += s[t, e] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)
        out = out + gate * clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def hyper_read(xs: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """xs [streams, T, W] -> the sublayer's input, a weighted sum of the streams."""
    return torch.einsum("s,stw->tw", w_in, xs)


def hyper_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    return torch.einsum("st,sjw->tjw", mix, xs) + w_out[:, None, None] * y[None]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    xs = x[None].repeat(cfg["streams"], 1, 1)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = unit_rms(hyper_read(xs, w[p + "hc1.in"]), eps) * w[p + "norm1"]
        if layer["type"] == "attention":
            y = softmax_attention(h, w, p + "mix.", layer["mixer"], "half")
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, p + "mix.", layer["mixer"], eps)
        else:
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        xs = hyper_write(xs, y, w[p + "hc1.mix"], w[p + "hc1.out"])
        if layer.get("mlp") is not None:
            h = unit_rms(hyper_read(xs, w[p + "hc2.in"]), eps) * w[p + "norm2"]
            if layer["mlp"]["kind"] == "dense":
                y = dense_feed_forward(h, w, p + "mlp.")
            else:
                y = mixture_of_experts(h, w, p + "mlp.", layer["mlp"], margins)
            xs = hyper_write(xs, y, w[p + "hc2.mix"], w[p + "hc2.out"])
        if layers_out is not None:
            layers_out.append(xs.sum(dim=0))
    return (unit_rms(xs.sum(dim=0), eps) * w["final.norm"]) @ w["embed"].T


class PlainPotodra:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_weights(model_dir)
        self._memo: dict = {}

    def run(self, tokens: List[int]) -> Tuple[torch.Tensor, float]:
        """(logits, the smallest margin of any router's decision over the sequence; infinite without routers)."""
        key = tuple(tokens)
        if key not in self._memo:
            margins: list = []
            self._memo[key] = (forward(self.cfg, self.w, tokens, None, margins), min(margins, default=float("inf")))
        return self._memo[key]

    def logits(self, tokens: List[int]) -> torch.Tensor:
        return self.run(tokens)[0]

    def closest_call(self, tokens: List[int]) -> float:
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
