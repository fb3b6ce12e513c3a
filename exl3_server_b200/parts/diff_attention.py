"""Differential attention: every head holds two softmax attention maps over the same values, and the second map's
output is subtracted from the first's.

Per token ``q = Wq r`` (``heads x 2 x head_dim``, head by head as [map 1 | map 2]), ``k = Wk r`` (``kv_heads x 2 x
head_dim``), ``v = Wv r`` (``kv_heads x value_dim``); query head h reads key/value head ``h // (heads / kv_heads)``.
Each map of q and k gets the spec's position encoding (half-split rotary pairs over the first ``dims`` features of
the map).  Map i of head h: ``a_i = softmax(q_i . k_i * softmax_scale over the visible keys) v`` with the causal mask
and, when ``window`` > 0, only the last ``window`` keys.  Then::

    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda0        (one number for the layer)
    o      = a_1 - lambda * a_2
    o      = o / sqrt(mean(o^2) + norm_eps) * (1 - lambda0)   (per head, over its value_dim values, no weight)
    o      = o * sigmoid(Wg r)_h                              (``gate`` "head": one number per token and head)
    y      = Wo concat_h(o)

Parameters of the spec: ``value_dim``, ``lambda0``, ``norm_eps``, ``gate`` (``"head"`` or ``"none"``).  Tensors under
the mixer's prefix: ``q``, ``k``, ``v``, ``o``, ``lq1``, ``lk1``, ``lq2``, ``lk2`` and, with a gate, ``g``.

How it runs: the attention kernels know nothing of maps.  The cache keeps, per kv head, one key row with its two
maps side by side (``2 * head_dim`` features, padded to a multiple of 8) and one value row; every map of a query
head becomes a query head of its own, as wide as the key row and zero outside its map, so its dot product with the
key row is the map's score (``kernels.maps_prep`` rotates, widens and writes the cache).  The framework's attention
kernels then run ``2 * heads`` query heads over ``kv_heads`` key/value heads with the window as their parameter and
leave float32 outputs; ``kernels.diff_combine`` subtracts, norms and gates in float32.  Scores, softmax, lambda, the
subtraction and the norm are float32 in either element type.

In bfloat16, a key row of 64 or 128 features with values no wider is the shape of the tensor-core attention kernels:
the value row is then as wide as the key row, and the maps run through the same choice of kernels as the
``attention`` mixer's heads (tcgen05 prompts, TMA decode), whose bfloat16 outputs ``diff_combine`` reads.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .attention import BUSY_ITEMS, SPLIT_KEYS, Attention
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import position_class, register_mixer
from .spec import MixerSpec, PositionSpec

MAPS = 2


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class MapsAsHeads(Attention):
    """The ``attention`` mixer's choice of kernels for queries that are already prepared: ``heads`` here are the
    maps, all of the key row's width, over keys and values that are in the cache."""

    def __init__(self, spec: MixerSpec, scale: float, ctx: BuildContext):
        self.spec, self.scale, self.ctx = spec, scale, ctx


class DifferentialAttention:
    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int, int]:
        dv = int(spec.params.get("value_dim", 0)) or spec.head_dim
        return spec.heads, spec.kv_heads, spec.head_dim, dv

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, G, d, dv = cls._sizes(spec)
        out = [TensorSpec(prefix + "q", (H * MAPS * d, spec.width)), TensorSpec(prefix + "k", (G * MAPS * d, spec.width)),
               TensorSpec(prefix + "v", (G * dv, spec.width)), TensorSpec(prefix + "o", (spec.width, H * dv))]
        out += [TensorSpec(prefix + n, (d,)) for n in ("lq1", "lk1", "lq2", "lk2")]
        if spec.params.get("gate", "none") == "head":
            out.append(TensorSpec(prefix + "g", (H, spec.width)))
        return out

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, G, d, dv = self._sizes(spec)
        if H < 1 or G < 1 or H % G != 0:
            raise ValueError(f"differential attention: {H} heads cannot share {G} kv heads")
        p = spec.params
        self.spec, self.ctx = spec, ctx
        self.H, self.G, self.d, self.dv = H, G, d, dv
        self.row, self.v_row = pad8(MAPS * d), pad8(dv)
        self.as_heads: Optional[MapsAsHeads] = None
        if ctx.dtype == torch.bfloat16 and self.row in (64, 128) and dv <= self.row:
            self.v_row = self.row
            self.as_heads = MapsAsHeads(
                MixerSpec(kind="attention", width=spec.width, heads=H * MAPS, kv_heads=G, head_dim=self.row,
                          window=int(spec.window)), 0.0, ctx)
        self.eps = float(p.get("norm_eps", 1e-6))
        self.lambda0 = float(p["lambda0"])
        self.window = int(spec.window)
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else d ** -0.5
        self.gated = p.get("gate", "none") == "head"
        if p.get("gate", "none") not in ("none", "head"):
            raise ValueError(f"differential attention: gate must be 'none' or 'head', got {p.get('gate')!r}")
        names = ("q", "k", "v", "g") if self.gated else ("q", "k", "v")
        self.proj = Linear(torch.cat([tensors[prefix + n].to(ctx.dtype) for n in names], dim=0), None, ctx.dtype)
        dots = [float((tensors[prefix + a].double() * tensors[prefix + b].double()).sum())
                for a, b in (("lq1", "lk1"), ("lq2", "lk2"))]
        self.lam = math.exp(dots[0]) - math.exp(dots[1]) + self.lambda0
        wo = tensors[prefix + "o"].to(ctx.dtype)
        if self.v_row != dv:                                # the attention's rows are padded: zero columns for the pad
            wo = torch.nn.functional.pad(wo.view(spec.width, H, dv), (0, self.v_row - dv)).reshape(spec.width, -1)
        self.o = Linear(wo, None, ctx.dtype)
        pos = spec.position or PositionSpec(kind="none", dims=0)
        if pos.kind == "rope" and pos.params.get("layout", "half") != "half":
            raise ValueError("differential attention: only the half-split rotary layout")
        self.position = position_class(pos.kind)(pos, d, ctx)
        self.rot = int(self.position.spec.dims)
        if self.as_heads is not None:
            self.as_heads.scale = self.scale

    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(self.G, self.row, self.window, self.v_row if self.v_row != self.row else 0)

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if kv is None or not kv.owns:
            raise RuntimeError("differential attention needs a cache view of its own")
        H, G, d, dv = self.H, self.G, self.d, self.dv
        T = x.shape[0]
        proj = self.proj(x, out_dtype=self.proj.wide_dtype(T))
        q_off, k_off = 0, H * MAPS * d
        v_off = k_off + G * MAPS * d
        g_off = v_off + G * dv
        q = K.maps_prep(proj, q_off, k_off, v_off, H, G, MAPS, d, dv, self.rot,
                        self.position.table if self.rot else None, batch.tok_pos, batch.tok_seq, kv.block_table,
                        kv.page_size, self.ctx.dtype, kv.k, kv.v)
        a = self._attend(q, batch, kv)
        gate = proj[:, g_off:g_off + H] if self.gated else None
        y = K.diff_combine(a, self.v_row, gate, self.lam, self.eps, 1.0 - self.lambda0, H, dv, self.v_row,
                           self.ctx.dtype)
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def _attend(self, q: torch.Tensor, batch, kv) -> torch.Tensor:
        """Both maps of every head as ``2 * heads`` query heads: ``[T, heads * 2 * value row]``, float32 from the
        CUDA-core kernel, bfloat16 from the tensor-core ones."""
        T = q.shape[0]
        nh = self.H * MAPS
        if self.as_heads is not None:
            out = torch.empty((T, nh * self.v_row), dtype=q.dtype, device=q.device)
            self.as_heads.attend(q, out, batch, kv)
            return out
        out = torch.empty((T, nh * self.v_row), dtype=torch.float32, device=q.device)
        split = max(SPLIT_KEYS, kv.page_size)
        if split % kv.page_size:
            split = kv.page_size * (split // kv.page_size + 1)
        n = self._chunks(batch.max_kv_len, split)
        # bfloat16 with more work items than the GPU holds at once: chunks twice as long (float32 keeps one chunking
        # for every batch, so that its results do not depend on the batch at all)
        if self.ctx.dtype == torch.bfloat16 and T * self.G * n > BUSY_ITEMS:
            split *= 2
            n = self._chunks(batch.max_kv_len, split)
        scratch = None
        if n > 1:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, nh, self.v_row, n) // 4)
        K.attn_tokens_ex(q, q.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T, nh, self.G,
                         self.row, self.v_row, kv.page_size, self.window, 0, False, self.scale, split, n, scratch)
        return out

    def _chunks(self, max_kv_len: int, split: int) -> int:
        """The most pieces of ``split`` keys that a token's visible keys can touch."""
        n = (max_kv_len + split - 1) // split
        if self.window > 0:
            n = min(n, (self.window + split - 2) // split + 1)
        return max(1, n)

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()


register_mixer("diff_attention", DifferentialAttention)
