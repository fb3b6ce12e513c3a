"""Feed-forwards.

``swiglu``, the dense gated feed-forward: ``y = (silu(r Wg^T) * (r Wu^T)) Wd^T``
(src/model.cpp:583-586; the reference applies SiLU unconditionally).  Gate and
up projections are one fused matrix; the product ``silu(g) * u`` is float32
inside its kernel.

``dense``: ``y = act(r Wu^T) Wd^T`` with an activation named in the spec's
``params["activation"]``: ``xielu``, ``gelu`` (exact, by erf), ``gelu_tanh`` or ``relu2`` (the square of relu).  ``xielu`` has two learned numbers ``p, q`` (tensor
``act``): ``softplus(p) z^2 + z/2`` for ``z > 0`` and
``(1/2 + softplus(q)) (exp(z) - 1 - z) + z/2`` otherwise; it is computed in
float32 (from float32 results of the up projection where the projection's kernel has them); for steps of few
tokens it is the epilogue of the up projection's weight-streaming kernel.

``gated``: ``y = Wd (act(Wg r) * (Wu r))`` with the gate's activation named in ``params["activation"]`` (``silu``,
``gelu`` or ``gelu_tanh``); tensors ``gate``, ``up``, ``down``.  Gate and up are one matrix; the product is float32
inside its kernel.

``clamped_glu``: ``y = Wd (g sigmoid(alpha g) (u + 1))`` with ``g = min(Wg r, limit)`` and ``u = clamp(Wu r, -limit,
limit)``; parameters ``limit`` and ``alpha`` (1.702 unless given); tensors ``gate``, ``up``, ``down``, no biases.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import FeedForwardSpec


class SwiGLU:
    @staticmethod
    def tensor_specs(spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        out = [
            TensorSpec(prefix + "gate_proj.weight", (spec.inner, spec.width)),
            TensorSpec(prefix + "up_proj.weight", (spec.inner, spec.width)),
            TensorSpec(prefix + "down_proj.weight", (spec.width, spec.inner)),
        ]
        for name, n in (("gate_proj", spec.inner), ("up_proj", spec.inner), ("down_proj", spec.width)):
            out.append(TensorSpec(prefix + name + ".bias", (n,), optional=True, init="zeros"))
        return out

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        wg = tensors[prefix + "gate_proj.weight"].to(ctx.dtype)
        wu = tensors[prefix + "up_proj.weight"].to(ctx.dtype)
        bg, bu = tensors.get(prefix + "gate_proj.bias"), tensors.get(prefix + "up_proj.bias")
        z = torch.zeros(spec.inner, dtype=ctx.dtype, device=wg.device)
        has_bias = bg is not None or bu is not None
        bg = bg.to(ctx.dtype) if bg is not None else z
        bu = bu.to(ctx.dtype) if bu is not None else z
        # Rows in eights: eight gate rows, then the eight up rows of the same
        # features.  A 16-row tile of the decode projection then holds both halves
        # of eight features and applies silu(gate) * up before it writes.
        self.interleave = 8 if spec.inner % 8 == 0 else 0
        if self.interleave:
            n = spec.inner // 8
            w = torch.stack([wg.view(n, 8, -1), wu.view(n, 8, -1)], dim=1).reshape(2 * spec.inner, -1)
            b = torch.stack([bg.view(n, 8), bu.view(n, 8)], dim=1).reshape(-1) if has_bias else None
        else:
            w = torch.cat([wg, wu], dim=0)
            b = torch.cat([bg, bu]) if has_bias else None
        self.gate_up = Linear(w, b, ctx.dtype)
        self.down = Linear(tensors[prefix + "down_proj.weight"], tensors.get(prefix + "down_proj.bias"), ctx.dtype)

    takes_then = True       # the last projection may fold its output into the residual (NormAfter)
    takes_raw = True        # the first projection takes a norm's output in two pieces (RawNormed)

    def forward(self, x: torch.Tensor, batch, then=None) -> torch.Tensor:
        if self.interleave and self.gate_up.fuses_gate():
            return self.down(self.gate_up.gated(x), then=then)
        return self.down(K.silu_mul(self.gate_up(x), interleave=self.interleave), then=then)

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


def _xielu(z: torch.Tensor, tensors, out_dtype):
    return K.xielu(z, tensors["act"], out_dtype)


def _xielu_prepare(tensors) -> None:
    """softplus(p) and 1/2 + softplus(q), worked out once (float64) from the two stored numbers, when the model is built."""
    p, q = (float(v) for v in tensors["act"].detach().double().cpu())
    sp = lambda v: v if v > 30.0 else math.log1p(math.exp(v))
    tensors["act.constants"] = (sp(p), 0.5 + sp(q))


def _xielu_fused(linear: Linear, x: torch.Tensor, tensors, out_dtype):
    """The up projection with the activation in its epilogue, or None where its kernel has none."""
    return linear.xielu(x, *tensors["act.constants"], out_dtype)


def _gelu(z: torch.Tensor, tensors, out_dtype):
    return K.activation(z, out_dtype, "gelu")


def _gelu_tanh(z: torch.Tensor, tensors, out_dtype):
    return K.activation(z, out_dtype, "gelu_tanh")


def _relu2(z: torch.Tensor, tensors, out_dtype):
    return K.activation(z, out_dtype, "relu2")


def _relu2_fused(linear: Linear, x: torch.Tensor, tensors, out_dtype):
    return linear.gelu(x, out_dtype, relu2=True)


def _gelu_fused(linear: Linear, x: torch.Tensor, tensors, out_dtype):
    return linear.gelu(x, out_dtype, tanh=False)


def _gelu_tanh_fused(linear: Linear, x: torch.Tensor, tensors, out_dtype):
    return linear.gelu(x, out_dtype, tanh=True)


def _no_prepare(tensors) -> None:
    return None


# name -> (parameter tensors as (suffix, shape), function(z, {suffix: tensor}, out_dtype),
#          function(linear, x, {suffix: tensor}, out_dtype) -> activated projection or None,
#          function({suffix: tensor}) called once when the part is built)
ACTIVATIONS = {"xielu": ((("act", (2,)),), _xielu, _xielu_fused, _xielu_prepare),
               "gelu": ((), _gelu, _gelu_fused, _no_prepare),             # z/2 (1 + erf(z / sqrt 2))
               "gelu_tanh": ((), _gelu_tanh, _gelu_tanh_fused, _no_prepare),   # z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
               "relu2": ((), _relu2, _relu2_fused, _no_prepare)}               # max(z, 0)^2


class DenseFeedForward:
    @staticmethod
    def _activation(spec: FeedForwardSpec):
        name = spec.params.get("activation", "xielu")
        try:
            return ACTIVATIONS[name]
        except KeyError:
            raise ValueError(f"dense feed-forward: no activation named {name!r}; known: {sorted(ACTIVATIONS)}") from None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        extra = cls._activation(spec)[0]
        return [TensorSpec(prefix + "up", (spec.inner, spec.width)),
                TensorSpec(prefix + "down", (spec.width, spec.inner))] + \
               [TensorSpec(prefix + name, shape) for name, shape in extra]

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        self.dtype = ctx.dtype
        extra, self.act, self.act_fused, prepare = self._activation(spec)
        self.act_tensors = {name: tensors[prefix + name].contiguous() for name, _ in extra}
        prepare(self.act_tensors)
        self.up = Linear(tensors[prefix + "up"], None, ctx.dtype)
        self.down = Linear(tensors[prefix + "down"], None, ctx.dtype)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        a = self.act_fused(self.up, x, self.act_tensors, self.dtype) if self.dtype == torch.bfloat16 else None
        if a is None:
            z = self.up(x, out_dtype=self.up.wide_dtype(x.shape[0]))
            a = self.act(z, self.act_tensors, self.dtype)
        return self.down(a, out_dtype=self.down.wide_dtype(x.shape[0]))

    def weight_bytes(self) -> int:
        return self.up.weight_bytes() + self.down.weight_bytes()


class GatedFeedForward:
    @staticmethod
    def tensor_specs(spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + "gate", (spec.inner, spec.width)), TensorSpec(prefix + "up", (spec.inner, spec.width)),
                TensorSpec(prefix + "down", (spec.width, spec.inner))]

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        self.dtype = ctx.dtype
        self.act = spec.params.get("activation", "silu")
        if self.act not in K.GATE_ACTIVATIONS:
            raise ValueError(f"gated feed-forward: no activation named {self.act!r}; known: {sorted(K.GATE_ACTIVATIONS)}")
        self.gate_up = Linear(torch.cat([tensors[prefix + "gate"].to(ctx.dtype), tensors[prefix + "up"].to(ctx.dtype)],
                                        dim=0), None, ctx.dtype)
        self.down = Linear(tensors[prefix + "down"], None, ctx.dtype)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        T = x.shape[0]
        return self.down(K.silu_mul(self.gate_up(x), act=self.act), out_dtype=self.down.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


class ClampedGLU:
    ALPHA = 1.702

    @staticmethod
    def tensor_specs(spec: FeedForwardSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + "gate", (spec.inner, spec.width)), TensorSpec(prefix + "up", (spec.inner, spec.width)),
                TensorSpec(prefix + "down", (spec.width, spec.inner))]

    def __init__(self, spec: FeedForwardSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        self.dtype = ctx.dtype
        self.limit = float(spec.params["limit"])
        self.alpha = float(spec.params.get("alpha", self.ALPHA))
        if not self.limit > 0:
            raise ValueError("clamped glu: the limit must be positive")
        self.gate_up = Linear(torch.cat([tensors[prefix + "gate"].to(ctx.dtype), tensors[prefix + "up"].to(ctx.dtype)],
                                        dim=0), None, ctx.dtype)
        self.down = Linear(tensors[prefix + "down"], None, ctx.dtype)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        T = x.shape[0]
        gu = self.gate_up(x, out_dtype=self.gate_up.wide_dtype(T))
        return self.down(K.clamped_glu(gu, self.limit, self.alpha, self.dtype), out_dtype=self.down.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("clamped_glu", ClampedGLU)
register_feed_forward("gated", GatedFeedForward)
register_feed_forward("dense", DenseFeedForward)
