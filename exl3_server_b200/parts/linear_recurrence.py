"""Mixers that keep a matrix state per head instead of keys and values (``csrc/linear_scan.cu``).

Both walk ``S <- decay * S + k_t v_t^T`` with ``S [dk, dv]`` per (sequence, head) in float32, kept in the cache's
per-sequence state (zero when a sequence starts), so a prompt cut into steps in any way, and token-by-token
decoding, walk the same chain (rows of many tokens run as chunks side by side, joined through the recurrence's
linearity, which changes roundings only).

``retention``: one fixed decay per head, no softmax and no denominator.  ``q, k`` (``heads x dk``) get the spec's
position encoding, ``k`` is multiplied by ``dk^(-1/2)`` after it; ``S_t = decay_h S_(t-1) + k_t v_t^T``,
``o_t = S_t^T q_t``; each head's ``o`` is divided by its root mean square, the heads are concatenated, multiplied by
``silu(Wg r)`` and projected by ``Wo``.  Parameters: ``key_dim``, ``value_dim``, ``decay`` (a list, one per head),
``norm_eps``.  Tensors: ``q``, ``k``, ``v``, ``g``, ``o``.

``wkv``: a decay per token and key channel that the token itself decides, and a bonus for the current token.  With
``r'`` the mixer's input of the token before (zeros before the first; part of the state), each of five inputs is its
own blend ``r + (r' - r) * mu_s``; ``r_t, k_t, v_t`` and the gate ``silu(.)`` are projections of theirs,
``w_t = exp(-exp(W2 tanh(W1 blend_w) + w0))``; per head ``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t``, then
``S_t = diag(w_t) S_(t-1) + k_t v_t^T``; each head's ``o`` divided by its root mean square, times a weight, times
the gate, then ``Wo``.  Parameters: ``key_dim`` (= value size), ``norm_eps``; the rank of ``W1, W2`` is whatever the
checkpoint has.  Tensors: ``mu.r``, ``mu.k``, ``mu.v``, ``mu.g``, ``mu.w``, ``r``, ``k``, ``v``, ``g``, ``w1``,
``w2``, ``w0``, ``u``, ``norm``, ``o``.

``lightning``: the same chain as ``retention`` with activations in place of positions: ``q, k = silu(Wq r),
silu(Wk r)`` (``heads x dk``), ``v = silu(Wv r)`` (``heads x dv``), no factor on the keys; ``S_t = decay_h S_(t-1) +
k_t v_t^T``, ``o_t = S_t^T q_t``; the concatenated heads are divided by their root mean square TOGETHER and
multiplied by a weight, then by ``sigmoid(Wg r)``, and projected by ``Wo``.  Parameters: ``key_dim``, ``value_dim``,
``decay`` (one per head), ``norm_eps``.  Tensors: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``.

Decays, their exponentials, the bonus, the state, the rotation and the per-head norms are float32; the projections
are the model's type.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import position_class, register_mixer
from .spec import MixerSpec, PositionSpec


def _scan_scratch(batch, T: int, heads: int, dk: int, dv: int):
    need = K.linear_scan_scratch_bytes(batch.n_rows, T, heads, dk, dv, batch.max_new)
    return batch.workspace.plain(need // 4) if need else None


class Retention:
    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int]:
        dk = int(spec.params["key_dim"])
        return spec.heads, dk, int(spec.params.get("value_dim", 0)) or dk

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, dk, dv = cls._sizes(spec)
        return [TensorSpec(prefix + "q", (H * dk, spec.width)), TensorSpec(prefix + "k", (H * dk, spec.width)),
                TensorSpec(prefix + "v", (H * dv, spec.width)), TensorSpec(prefix + "g", (H * dv, spec.width)),
                TensorSpec(prefix + "o", (spec.width, H * dv))]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, dk, dv = self._sizes(spec)
        decay = [float(x) for x in spec.params["decay"]]
        if H < 1 or len(decay) != H:
            raise ValueError(f"retention: {len(decay)} decays for {H} heads")
        self.spec, self.ctx = spec, ctx
        self.H, self.dk, self.dv = H, dk, dv
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(ctx.device)
        self._w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("q", "k", "v", "g")], dim=0)
        self.n_proj = self._w.shape[0]
        self.proj: Optional[Linear] = None
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)
        pos = spec.position or PositionSpec(kind="none", dims=0)
        self.position = position_class(pos.kind)(pos, dk, ctx)
        self.rot = int(self.position.spec.dims)

    def input_weight(self):
        return self._w, None

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.H, self.dk, self.dv), torch.float32)

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if self.proj is None:
            self.proj = Linear(self._w, None, self.ctx.dtype)
        return self.forward_projected(self.proj(x, out_dtype=self.proj.wide_dtype(x.shape[0])), 0, batch, kv, state)

    def forward_projected(self, proj: torch.Tensor, off: int, batch, kv, state) -> torch.Tensor:
        """``proj [T, *]`` holds this mixer's ``[q | k | v | g]`` from column ``off`` on."""
        if state is None:
            raise RuntimeError("retention needs its per-sequence state")
        H, dk, dv = self.H, self.dk, self.dv
        T = proj.shape[0]
        # rotation and the keys' factor in float32: what enters the recurrence is not rounded again
        q, k = K.qk_prep(proj, off, off + H * dk, -1, H, H, dk, 0, dk, 0, 0, None, None, self.eps, self.rot,
                         self.position.layout_code, self.position.table if self.rot else None, self.position.mscale,
                         float(dk) ** -0.5, None, batch.tok_pos, batch.tok_seq, None, 0, torch.float32, None, None,
                         k_dtype=torch.float32)
        v = proj[:, off + 2 * H * dk: off + 2 * H * dk + H * dv]
        g = proj[:, off + 2 * H * dk + H * dv: off + 2 * H * dk + 2 * H * dv]
        o = K.linear_scan(1, q, k, v, state, batch.slot_ids, batch.row_start, batch.n_rows, H, dk, dv, batch.max_new,
                          decay=self.decay, scratch=_scan_scratch(batch, T, H, dk, dv))
        y = K.head_norm_gate(o, None, g, self.eps, H, dv, self.ctx.dtype)
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self._w.numel() * self._w.element_size() + self.o.weight_bytes()


class Lightning:
    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int]:
        dk = int(spec.params["key_dim"])
        return spec.heads, dk, int(spec.params.get("value_dim", 0)) or dk

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, dk, dv = cls._sizes(spec)
        return [TensorSpec(prefix + "q", (H * dk, spec.width)), TensorSpec(prefix + "k", (H * dk, spec.width)),
                TensorSpec(prefix + "v", (H * dv, spec.width)), TensorSpec(prefix + "g", (H * dv, spec.width)),
                TensorSpec(prefix + "o", (spec.width, H * dv)), TensorSpec(prefix + "norm", (H * dv,), init="ones")]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, dk, dv = self._sizes(spec)
        decay = [float(x) for x in spec.params["decay"]]
        if H < 1 or len(decay) != H:
            raise ValueError(f"lightning: {len(decay)} decays for {H} heads")
        self.spec, self.ctx = spec, ctx
        self.H, self.dk, self.dv = H, dk, dv
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(ctx.device)
        self.proj = Linear(torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("q", "k", "v", "g")], dim=0), None,
                           ctx.dtype)
        self.norm_w = tensors[prefix + "norm"].float().contiguous()
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.H, self.dk, self.dv), torch.float32)

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if state is None:
            raise RuntimeError("lightning needs its per-sequence state")
        H, dk, dv = self.H, self.dk, self.dv
        T = x.shape[0]
        proj = self.proj(x, out_dtype=self.proj.wide_dtype(T))
        q, k = proj[:, :H * dk], proj[:, H * dk:2 * H * dk]
        v = proj[:, 2 * H * dk:2 * H * dk + H * dv]
        g = proj[:, 2 * H * dk + H * dv:]
        # SiLU in float32 as the scan reads its inputs: what enters the recurrence is not rounded again
        o = K.linear_scan(1, q, k, v, state, batch.slot_ids, batch.row_start, batch.n_rows, H, dk, dv, batch.max_new,
                          decay=self.decay, scratch=_scan_scratch(batch, T, H, dk, dv), in_act="silu")
        # all heads are normed together: one "head" of H * dv values
        y = K.head_norm_gate(o, self.norm_w, g, self.eps, 1, H * dv, self.ctx.dtype, gate_kind="sigmoid")
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()


class WKV:
    BLENDS = ("r", "k", "v", "g", "w")

    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int]:
        return spec.heads, int(spec.params["key_dim"])

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, d = cls._sizes(spec)
        W = spec.width
        rank = int(spec.params.get("decay_rank", 0)) or -1          # -1: whatever the checkpoint has
        free = int(spec.params.get("decay_rank", 0)) or 16
        return [TensorSpec(prefix + "mu." + s, (W,)) for s in cls.BLENDS] + [
            TensorSpec(prefix + "r", (H * d, W)), TensorSpec(prefix + "k", (H * d, W)),
            TensorSpec(prefix + "v", (H * d, W)), TensorSpec(prefix + "g", (H * d, W)),
            TensorSpec(prefix + "w1", (rank, W), free_dim=free), TensorSpec(prefix + "w2", (H * d, rank), free_dim=free),
            TensorSpec(prefix + "w0", (H * d,)), TensorSpec(prefix + "u", (H, d)),
            TensorSpec(prefix + "norm", (H * d,), init="ones"), TensorSpec(prefix + "o", (W, H * d))]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, d = self._sizes(spec)
        if H < 1 or d < 1:
            raise ValueError("wkv: heads and key_dim must be positive")
        self.spec, self.ctx = spec, ctx
        self.H, self.d = H, d
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        self.mu = torch.stack([tensors[prefix + "mu." + s].float() for s in self.BLENDS]).contiguous()
        self.r = Linear(tensors[prefix + "r"], None, ctx.dtype)
        self.k = Linear(tensors[prefix + "k"], None, ctx.dtype)
        self.v = Linear(tensors[prefix + "v"], None, ctx.dtype)
        self.g = Linear(tensors[prefix + "g"], None, ctx.dtype)
        self.w1 = Linear(tensors[prefix + "w1"], None, ctx.dtype)
        self.w2 = Linear(tensors[prefix + "w2"], None, ctx.dtype)
        if self.w1.out_features != self.w2.in_features:
            raise ValueError(f"wkv: {prefix}w1 and {prefix}w2 disagree about their rank")
        self.w0 = tensors[prefix + "w0"].float().contiguous()
        self.u = tensors[prefix + "u"].float().contiguous()
        self.norm_w = tensors[prefix + "norm"].float().contiguous()
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self):
        # the input of the token before, and the matrix state
        return (StateRequest((self.spec.width,), torch.float32), StateRequest((self.H, self.d, self.d), torch.float32))

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if state is None:
            raise RuntimeError("wkv needs its per-sequence state")
        before, S = state
        H, d = self.H, self.d
        T = x.shape[0]
        dt = self.ctx.dtype
        blends = K.token_shift(x, self.mu, before, batch.tok_seq, batch.row_start, batch.slot_ids, dt)
        r = self.r(blends[0], out_dtype=self.r.wide_dtype(T))
        k = self.k(blends[1], out_dtype=self.k.wide_dtype(T))
        v = self.v(blends[2], out_dtype=self.v.wide_dtype(T))
        g = self.g(blends[3], out_dtype=self.g.wide_dtype(T))
        low = K.activation(self.w1(blends[4], out_dtype=self.w1.wide_dtype(T)), dt, "tanh")
        wraw = self.w2(low, out_dtype=self.w2.wide_dtype(T))
        o = K.linear_scan(0, r, k, v, S, batch.slot_ids, batch.row_start, batch.n_rows, H, d, d, batch.max_new,
                          wraw=wraw, w0=self.w0, u=self.u, scratch=_scan_scratch(batch, T, H, d, d))
        y = K.head_norm_gate(o, self.norm_w, g, self.eps, H, d, dt)
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def weight_bytes(self) -> int:
        return sum(l.weight_bytes() for l in (self.r, self.k, self.v, self.g, self.w1, self.w2, self.o))


register_mixer("retention", Retention)
register_mixer("wkv", WKV)
register_mixer("lightning", Lightning)
