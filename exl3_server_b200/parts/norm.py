"""RMSNorm fused with the residual add.

``r = h * rsqrt(mean(h^2) + eps) * w`` with the weight multiplying directly
(no ``1 + w``), as the reference's ``mx::fast::rms_norm`` calls use it
(src/model.cpp:556, 582, 589).  The sum of squares, the reciprocal root and the
residual add ``h += scale * y`` are float32.

The same norm also serves layers that norm a sublayer's output instead of its
input (``add_normed``: ``h += rmsnorm(y) * w``; the ``outnorm`` and ``sandwich`` arrangements).

Parameters of the spec: ``suffix`` (the tensor's name after the prefix), ``one_plus`` (the stored weight lies
around zero and the factor is ``1 + w``) and ``scale`` (a constant on the norm's output, such as a multiplier of
the residual branch).

``rms_streams``: the RMS norm of a residual of several streams (``params["streams"]``, see ``parts/block.py``,
arrangement ``hyper``): the streams are summed and the sum is normed, in one kernel.

``tanh``: a norm that computes no statistics, ``r = tanh(alpha * h) * w + b`` with one learned number ``alpha`` and
the vectors ``w`` and ``b`` (tensors: the prefix itself, or prefix + ``suffix``, for ``w``; that name + ``.b`` and
+ ``.alpha``).  Float32 throughout.  The spec's ``eps`` is not used.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, ReadyNormed, ResidualStream
from .registry import register_norm
from .spec import NormSpec


class RMSNorm:
    @staticmethod
    def tensor_specs(spec: NormSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + spec.params.get("suffix", "weight"), (spec.width,), init="ones")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        w = tensors[prefix + spec.params.get("suffix", "weight")]     # the tensor's name is prefix + suffix
        one_plus, scale = bool(spec.params.get("one_plus", False)), float(spec.params.get("scale", 1.0))
        if one_plus or scale != 1.0:
            # a weight stored around zero (the factor is 1 + w) and a constant on the norm's output: both folded
            # into one float32 weight when the model is built
            w = ((w.float() + 1.0) if one_plus else w.float()) * scale
        # a weight stored in 32-bit stays 32-bit; the kernel reads either
        self.weight = w.contiguous() if w.dtype == torch.float32 else w.to(ctx.dtype).contiguous()
        self.out_dtype = ctx.dtype

    offers_raw = True

    def add_norm(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                 out_scale: float = 1.0, raw_ok: bool = False):
        """``raw_ok``: the caller's next projection takes a ``RawNormed`` (the output in two pieces, left by the
        projection before this norm) as well as a tensor."""
        left = stream.take_normed(self)
        if left is not None:
            if rows is None and raw_ok and out_scale == 1.0 and not isinstance(left, ReadyNormed):
                return left
            return left.materialize(out_scale, rows)
        y, s = stream.take()
        if y is not None:
            stream.act = None
        return K.add_rmsnorm(stream.h, y, s, self.weight, self.spec.eps, self.out_dtype,
                             out_scale=out_scale, rows=rows)

    def add_normed(self, stream: ResidualStream, y: Optional[torch.Tensor], want_x: bool = True) -> Optional[torch.Tensor]:
        """The norm on a sublayer's OUTPUT: ``h += y * rsqrt(mean(y^2) + eps) * w`` in float32; returns the new
        residual in the activation type, which the next sublayer reads (``h`` itself in the float32 path).  With
        ``y`` None nothing is added and the residual is only handed over.  ``want_x`` False: nothing is returned
        (the next sublayer reads a norm of the residual, not the residual)."""
        if stream.pending is not None:
            raise RuntimeError("the residual stream holds an output that was not folded in")
        stream.normed = None
        if not want_x:
            stream.act = None
            K.norm_add(stream.h, y, self.weight, self.spec.eps, None)
            return None
        x_dtype = None if self.out_dtype == torch.float32 else self.out_dtype
        x = K.norm_add(stream.h, y, self.weight if y is not None else None, self.spec.eps, x_dtype)
        stream.act = x if x is not None else stream.h
        return stream.act

    def add_normed_then(self, stream: ResidualStream, y: torch.Tensor, then_norm) -> None:
        """``add_normed`` and, in the same kernel, the output of ``then_norm`` (the next sublayer's input norm) over
        the new residual, left in the stream for ``then_norm.add_norm`` to pick up."""
        if stream.pending is not None:
            raise RuntimeError("the residual stream holds an output that was not folded in")
        x = K.norm_add_norm(stream.h, y, self.weight, self.spec.eps, then_norm.weight, then_norm.spec.eps,
                            then_norm.out_dtype)
        stream.act = None
        stream.normed = (then_norm, ReadyNormed(x))

    def fuse_args(self):
        """``(weight, eps, width)`` for a projection kernel that prepares this norm (see ``NormAfter``)."""
        return self.weight, self.spec.eps, self.spec.width

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()


class StreamsRMSNorm(RMSNorm):
    """``r = rmsnorm(sum_s x_s) * w`` over a residual ``[T, streams * width]`` (or ``[T, width]``, when nothing has
    widened it yet: equal streams)."""

    offers_raw = False

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        super().__init__(spec, tensors, prefix, ctx)
        self.streams = int(spec.params.get("streams", 1))
        self._ones = torch.ones(self.streams, dtype=torch.float32, device=self.weight.device)

    def add_norm(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                 raw_ok: bool = False):
        if out_scale != 1.0 or stream.pending is not None:
            raise ValueError("streams norm: no constant on the output and nothing pending in the stream")
        S, W = self.streams, self.spec.width
        if stream.h.shape[1] == W and S > 1:
            # equal streams: their sum is S times the row; the norm of a multiple differs from the row's own only
            # through eps, so the factor goes in as the read weights
            ones = self._ones
            wide = torch.empty((stream.h.shape[0], S * W), dtype=torch.float32, device=stream.h.device)
            _, r = K.hyper_step(stream.h, S, None, None, None, ones, self.weight, self.spec.eps, self.out_dtype, out=wide)
            if rows is not None:
                r = r.index_select(0, rows.long())
            return r
        return K.hyper_step(stream.h, S, None, None, None, self._ones, self.weight, self.spec.eps, self.out_dtype,
                            rows=rows)[1]


class DynamicTanhNorm:
    @staticmethod
    def _name(spec: NormSpec, prefix: str) -> str:
        return prefix + spec.params.get("suffix", "")

    @classmethod
    def tensor_specs(cls, spec: NormSpec, prefix: str) -> List[TensorSpec]:
        n = cls._name(spec, prefix)
        return [TensorSpec(n, (spec.width,), init="ones"), TensorSpec(n + ".b", (spec.width,)),
                TensorSpec(n + ".alpha", (), init="ones")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        n = self._name(spec, prefix)
        self.spec = spec
        self.weight = tensors[n].float().contiguous()
        self.bias = tensors[n + ".b"].float().contiguous()
        self.alpha = tensors[n + ".alpha"].float().reshape(1).contiguous()
        self.out_dtype = ctx.dtype
        self._ones: Optional[torch.Tensor] = None

    def tanh_args(self):
        """``(w, b, alpha)`` for a kernel that applies this norm together with something else."""
        return self.weight, self.bias, self.alpha

    def add_norm(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                 raw_ok: bool = False):
        if out_scale != 1.0:
            raise ValueError("tanh norm: no constant on the output (fold it into the weight and the bias)")
        left = stream.take_normed(self)
        if left is not None:
            return left.materialize(1.0, rows)
        y, s = stream.take()
        if y is not None:
            stream.act = None
            if self._ones is None:
                self._ones = torch.ones_like(self.weight)
            if rows is None:
                return K.tanh_norm_add(stream.h, y, None, self._ones, None, s, [self.tanh_args()], self.out_dtype)[0]
            K.tanh_norm_add(stream.h, y, None, self._ones, None, s, [], self.out_dtype)
        return K.tanh_norm_add(stream.h, None, None, None, None, 1.0, [self.tanh_args()], self.out_dtype, rows=rows)[0]

    def weight_bytes(self) -> int:
        return 4 * (self.weight.numel() + self.bias.numel() + 1)


register_norm("rms", RMSNorm)
register_norm("rms_streams", StreamsRMSNorm)
register_norm("tanh", DynamicTanhNorm)
