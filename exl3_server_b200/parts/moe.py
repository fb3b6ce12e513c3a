"""A routed feed-forward (mixture of experts) with optional identity experts and a shared expert.

The router has ``experts + identity`` outputs: ``z = Wr r`` in float32, scores ``s = softmax(z)`` over all of them.
The choice is made by ``c = s + correction`` (a stored vector); the outputs form ``groups`` equal groups of
neighbours, a group's score is its largest ``c``, and only outputs of the ``keep`` best groups can be chosen (the
others count as minus infinity); the ``top`` largest ``c`` among them are the token's picks.  A pick's weight is its
score ``s`` (without the correction) times ``scale``; weights are not renormalised.  Picks below ``experts`` are
small feed-forwards ``Wd_e act(Wu_e r)`` without biases (tensors ``e<i>.up``, ``e<i>.down``); the last ``identity``
outputs have no tensors and stand for the input ``r`` itself.  The output is the weighted sum of the picks, plus, when
the spec has ``shared_inner``, a shared expert of the same form (``shared.up``, ``shared.down``) that every token
runs, times ``sigmoid(w_sg . r)`` (``shared.sg``, one number per token).

Parameters of the spec: ``experts``, ``identity``, ``top``, ``scale``, ``groups``, ``keep``, ``activation`` (``gelu``,
``gelu_tanh`` or ``silu``), ``score`` (``softmax`` or ``sigmoid``), ``group_score`` (``max``, or ``top2``: a group's
score is the sum of its two largest choice scores), ``shared_inner`` (0: none); ``inner`` is an expert's hidden size.
``expert`` = ``"clamped_glu"`` makes the experts (and the shared one) gated with a bounded gate, ``Wd (g sigmoid(alpha
g) (u + 1))``, ``g = min(Wg r, limit)``, ``u = clamp(Wu r, -limit, limit)`` (tensors ``e<i>.gate``, ``e<i>.up``,
``e<i>.down``; parameters ``limit``, ``shared_limit``, ``alpha``): gate and up are one stacked matrix per expert, the
activation a kernel of its own between the two grouped products.  Tensors: ``router [experts + identity, width]``, ``correction [experts + identity]`` and the
experts'.

How it runs (``csrc/moe.cu``): the router kernel also computes the shared expert's gate (its vector is one more row
of the router's float32 matrix); a one-block kernel orders the step's (token, pick) pairs by expert into tiles, on the
device, so a step is the same list of launches whatever the router chose (it can be part of a recorded graph); the
experts' weights are stacked ``[experts, out, in]`` and both projections are grouped products over the tiles; the
last kernel sums picks, identity picks and the gated shared expert in float32.  Which product runs depends on the
step only through its number of pairs: in bfloat16, few pairs (decode) take the kernel that reads each expert's
matrix once with a warp per output feature, many pairs (prompts) are gathered into the plan's order and go through
the tcgen05 grouped product; float32, and sizes those two do not take, use the CUDA-core tiles.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext
from .ffn import ClampedGLU, DenseFeedForward
from .registry import register_feed_forward
from .spec import FeedForwardSpec


FEW_PAIRS = 128       # up to here the few-row product; from MANY_PAIRS on the tensor cores
MANY_PAIRS = 512


class RoutedFeedForward:
    @staticmethod
    def _sizes(spec: FeedForwardSpec):
        p = spec.params
        return int(p["experts"]), int(p.get("identity", 0)), int(p.get("shared_inner", 0))

    @staticmethod
    def _clamped(spec: FeedForwardSpec) -> bool:
        return spec.params.get("expert", "dense") == "clamped_glu"

    @classmethod
    def _shared_spec(cls, spec: FeedForwardSpec, inner: int) -> FeedForwardSpec:
        if cls._clamped(spec):
            return FeedForwardSpec(kind="clamped_glu", width=spec.width, inner=inner,
                                   params={"limit": spec.params.get("shared_limit", spec.params["limit"]),
                                           "alpha": spec.params.get("alpha", ClampedGLU.ALPHA)})
        return FeedForwardSpec(kind="dense", width=spec.width, inner=inner,
                               params={"activation": spec.params.get("activation", "gelu")})

    @classmethod
    def _shared_class(cls, spec: FeedForwardSpec):
        return ClampedGLU if cls._clamped(spec) else DenseFeedForward

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        E, I, shared = cls._sizes(spec)
        out = [TensorSpec(prefix + "router", (E + I, spec.width)), TensorSpec(prefix + "correction", (E + I,))]
        for e in range(E):
            if cls._clamped(spec):
                out.append(TensorSpec(f"{prefix}e{e}.gate", (spec.inner, spec.width)))
            out += [TensorSpec(f"{prefix}e{e}.up", (spec.inner, spec.width)),
                    TensorSpec(f"{prefix}e{e}.down", (spec.width, spec.inner))]
        if shared:
            out += cls._shared_class(spec).tensor_specs(cls._shared_spec(spec, shared), prefix + "shared.")
            out.append(TensorSpec(prefix + "shared.sg", (1, spec.width)))
        return out

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        E, I, shared = self._sizes(spec)
        p = spec.params
        self.spec, self.dtype = spec, ctx.dtype
        self.E, self.I = E, I
        self.top, self.scale = int(p["top"]), float(p.get("scale", 1.0))
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep", 1))
        self.act, self.score = p.get("activation", "gelu"), p.get("score", "softmax")
        self.group_score = p.get("group_score", "max")
        self.clamped = self._clamped(spec)
        if self.clamped:
            self.act = "none"                  # the bounded gate is applied between the two products
            self.limit, self.alpha = float(p["limit"]), float(p.get("alpha", ClampedGLU.ALPHA))
        if self.act not in K.MOE_ACTIVATIONS or self.score not in K.MOE_SCORES or self.group_score not in K.MOE_GROUP_SCORES:
            raise ValueError(f"routed feed-forward: unknown activation {self.act!r}, score {self.score!r} or group "
                             f"score {self.group_score!r}")
        n = E + I
        if n < 1 or n % self.groups != 0 or not 1 <= self.keep <= self.groups or \
                not 1 <= self.top <= self.keep * (n // self.groups):
            raise ValueError(f"routed feed-forward: {n} outputs, {self.groups} groups, keep {self.keep}, top {self.top}")
        rows = [tensors[prefix + "router"].float()]
        self.shared = None
        if shared:
            self.shared = self._shared_class(spec)(self._shared_spec(spec, shared), tensors, prefix + "shared.", ctx)
            rows.append(tensors[prefix + "shared.sg"].float().reshape(1, spec.width))
        self.router = torch.cat(rows, dim=0).contiguous()             # float32: the router is computed in 32 bits
        self.correction = tensors[prefix + "correction"].float().contiguous()
        self.w_up = self.w_down = None
        if E:
            if self.clamped:                   # [gate; up] rows of every expert
                self.w_up = torch.stack([torch.cat([tensors[f"{prefix}e{e}.gate"].to(ctx.dtype),
                                                    tensors[f"{prefix}e{e}.up"].to(ctx.dtype)], dim=0)
                                         for e in range(E)]).contiguous()
            else:
                self.w_up = torch.stack([tensors[f"{prefix}e{e}.up"].to(ctx.dtype) for e in range(E)]).contiguous()
            self.w_down = torch.stack([tensors[f"{prefix}e{e}.down"].to(ctx.dtype) for e in range(E)]).contiguous()

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        idx, wt, gate = K.moe_route(x, self.router, self.correction, self.E + self.I, 1 if self.shared else 0,
                                    self.groups, self.keep, self.top, self.scale, self.score, self.group_score)
        y = None
        if self.E:
            y = self._experts(x, idx)
        s = self.shared.forward(x, batch) if self.shared is not None else None
        return K.moe_combine(y, idx, wt, x, s, gate, self.E)

    def _experts(self, x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """float32 ``[pairs, width]``: every planned pair's expert output at the pair's own place."""
        pairs = idx.numel()
        width, inner = self.w_up.shape[2], self.w_down.shape[2]
        glu = (lambda mid: K.clamped_glu(mid, self.limit, self.alpha, self.dtype)) if self.clamped else (lambda mid: mid)
        vec = self.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and width % 8 == 0 and inner % 8 == 0 and \
            x.stride(0) % 8 == 0
        if vec and pairs >= MANY_PAIRS and K.moe_tc_supported(self.dtype, inner, width):
            order, plan = K.moe_plan(idx, self.E, K.moe_tile_rows("tc"))
            xs = K.moe_gather(x, self.top, order, plan)
            mid = glu(K.moe_gemm_tc(xs, self.w_up, order, plan, self.dtype, act=self.act))
            return K.moe_gemm_tc(mid, self.w_down, order, plan, torch.float32)
        if vec and pairs <= FEW_PAIRS:
            order, plan = K.moe_plan(idx, self.E, K.moe_tile_rows("few"))
            mid = glu(K.moe_gemv(x, self.top, self.w_up, order, plan, self.dtype, act=self.act))
            return K.moe_gemv(mid, 1, self.w_down, order, plan, torch.float32)
        order, plan = K.moe_plan(idx, self.E)
        mid = glu(K.moe_gemm(x, self.top, self.w_up, order, plan, self.dtype, act=self.act))
        return K.moe_gemm(mid, 1, self.w_down, order, plan, torch.float32)

    def untouched_bytes(self, tokens: int) -> int:
        """Bytes of experts' matrices that a step of ``tokens`` tokens is not expected to read when every router output
        is as likely a pick as any other (random weights): an output stays unpicked by a token with probability
        ``1 - top / outputs``."""
        if self.w_up is None:
            return 0
        per_expert = (self.w_up[0].numel() + self.w_down[0].numel()) * self.w_up.element_size()
        return int(self.E * per_expert * (1.0 - self.top / (self.E + self.I)) ** tokens)

    def weight_bytes(self) -> int:
        """Weight bytes a token's step reads at most: the router, the shared expert and ``top`` experts per token
        (a step of many tokens reads each expert once; this counts the matrices once)."""
        n = self.router.numel() * 4 + self.correction.numel() * 4
        if self.w_up is not None:
            n += (self.w_up.numel() + self.w_down.numel()) * self.w_up.element_size()
        if self.shared is not None:
            n += self.shared.weight_bytes()
        return n


register_feed_forward("routed", RoutedFeedForward)
