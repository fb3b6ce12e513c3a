"""Arrangements of a layer's parts.

``prenorm``: ``h += rho * mixer(norm1(h))`` then ``h += rho * ff(norm2(h))``
(src/model.cpp:556-586, with rho = 1 there).  The sublayer output is
multiplied by ``residual_scale`` and then added, in float32, inside the next
norm's kernel.

``outnorm``: the sublayers read the residual itself and the norm sits on their
output: ``h += norm1(mixer(h))`` then ``h += norm2(ff(h))``.  The norm, the add
(float32) and the cast of the new residual for the next sublayer are one kernel.
A layer of this kind may have no feed-forward at all.

``sandwich``: a norm on both sides of each sublayer: ``h += rho * norm1b(mixer(norm1(h)))`` then
``h += rho * norm2b(ff(norm2(h)))``.  The constant ``rho`` is a parameter of the output norms (their ``scale``), so
the second norm, the constant and the add (float32) are one kernel, as in ``outnorm``.

``side_by_side``: both sublayers read norms of the same residual and their outputs are added together, each times a
learned vector of its own (a layer scale): ``h += rho * (s1 * mixer(norm1(h)) + s2 * ff(norm2(h)))``.  The step, in
float32, and the two norms that the next block of this kind applies to the new residual are one kernel
(``kernels.tanh_norm_add``) when those norms are of the ``tanh`` kind; other norms run as kernels of their own.  The
vectors are tensors of the arrangement (names under ``mixer_scale`` and ``feed_forward_scale``).  A layer may have no
feed-forward.

``hyper``: hyper-connections.  The residual is ``streams`` rows per token, ``x_1 .. x_S``, all equal to the embedding at
the start.  Sublayer q (1: the mixer, 2: the feed-forward) reads ``u = sum_s a_q[s] x_s``, runs on ``norm_q(u)`` and
writes to every stream at once from the old ones, ``x_t <- sum_s M_q[s, t] x_s + b_q[t] y`` (``M_q`` indexed [from,
to]).  ``a_q``, ``b_q`` and ``M_q`` are tensors of the arrangement (names under ``hyper1`` / ``hyper2`` + ``.in``,
``.out``, ``.mix``).  A write and the read that follows it (the next sublayer's, or the next block's first) are one
float32 kernel (``kernels.hyper_step``), so a layer has as many element-wise kernels as a pre-norm layer has.  With
one stream, ``M = [[1]]`` and ``a = b = [1]`` this is ``prenorm``.  The model's last norm must be of the
``rms_streams`` kind (it sums the streams).  A layer may have no feed-forward.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import NormAfter, ResidualStream
from .registry import register_arrangement
from .spec import LayerSpec


class PreNormBlock:
    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    takes_after = True

    def forward(self, stream: ResidualStream, batch, kv, state, after=None) -> None:
        """``after``: the norm that the next block will apply first, if the caller knows it: the feed-forward's
        last projection may then apply it in its own kernel, as the mixer's may apply this block's second norm."""
        r = self._norm(self.mixer_norm, stream, self.mixer)
        self._run(self.mixer, (r, batch, kv, state), stream, self.feed_forward_norm)
        r = self._norm(self.feed_forward_norm, stream, self.feed_forward)
        self._run(self.feed_forward, (r, batch), stream, after)

    @staticmethod
    def _norm(norm, stream: ResidualStream, part):
        # a part whose first projection takes a norm's output in two pieces gets it that way when it is there
        if getattr(norm, "offers_raw", False) and getattr(part, "takes_raw", False):
            return norm.add_norm(stream, raw_ok=True)
        return norm.add_norm(stream)

    def _run(self, part, args, stream: ResidualStream, norm) -> None:
        then = None
        if norm is not None and getattr(part, "takes_then", False):
            then = NormAfter(stream, self.spec.residual_scale, norm)
            y = part.forward(*args, then=then)
        else:
            y = part.forward(*args)
        if then is None or not then.done:
            stream.push(y, self.spec.residual_scale)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm,
                                              self.feed_forward_norm) if hasattr(p, "weight_bytes"))


class OutNormBlock:
    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        if spec.residual_scale != 1.0:
            raise ValueError("outnorm: a scale on the sublayer's output would be undone by the norm")
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward              # None: the layer is its mixer only
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, stream: ResidualStream, batch, kv, state) -> None:
        x = stream.act if stream.act is not None and stream.pending is None else self.mixer_norm.add_normed(stream, None)
        x = self.mixer_norm.add_normed(stream, self.mixer.forward(x, batch, kv, state))
        if self.feed_forward is not None:
            self.feed_forward_norm.add_normed(stream, self.feed_forward.forward(x, batch))

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm)
                   if p is not None and hasattr(p, "weight_bytes"))


class SandwichBlock:
    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm, out_norms=(None, None)):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward              # None: the layer is its mixer only
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.mixer_out_norm, self.feed_forward_out_norm = out_norms
        if self.mixer_out_norm is None or (feed_forward is not None and self.feed_forward_out_norm is None):
            raise ValueError("sandwich: every sublayer needs a norm on its output")
        for n in (self.mixer_out_norm, self.feed_forward_out_norm):
            if n is not None and float(n.spec.params.get("scale", 1.0)) != float(spec.residual_scale):
                raise ValueError("sandwich: the output norms' scale must be the layer's residual scale")

    takes_after = True

    def forward(self, stream: ResidualStream, batch, kv, state, after=None) -> None:
        """``after``: the norm that the next block applies first, if the caller knows it: the kernel that adds this
        block's last sublayer to the residual then also computes that norm (as it does for this block's second
        sublayer)."""
        x = self.mixer_norm.add_norm(stream)
        y = self.mixer.forward(x, batch, kv, state)
        nxt = self.feed_forward_norm if self.feed_forward is not None else after
        self._add(self.mixer_out_norm, stream, y, nxt)
        if self.feed_forward is not None:
            x = self.feed_forward_norm.add_norm(stream)
            self._add(self.feed_forward_out_norm, stream, self.feed_forward.forward(x, batch), after)

    @staticmethod
    def _add(out_norm, stream: ResidualStream, y, then_norm) -> None:
        if then_norm is not None and hasattr(out_norm, "add_normed_then") and hasattr(then_norm, "weight"):
            out_norm.add_normed_then(stream, y, then_norm)
        else:
            out_norm.add_normed(stream, y, want_x=False)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm,
                                              self.mixer_out_norm, self.feed_forward_out_norm)
                   if p is not None and hasattr(p, "weight_bytes"))


class SideBySideBlock:
    takes_tensors = True      # built with the checkpoint's tensors (the layer-scale vectors)
    takes_next = True         # forward gets the block that runs next

    @staticmethod
    def tensor_specs(spec: LayerSpec) -> List[TensorSpec]:
        out = [TensorSpec(spec.names["mixer_scale"], (spec.mixer.width,), init="ones")]
        if spec.feed_forward is not None:
            out.append(TensorSpec(spec.names["feed_forward_scale"], (spec.mixer.width,), init="ones"))
        return out

    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm,
                 tensors: Dict[str, torch.Tensor]):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward              # None: the layer is its mixer only
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm if feed_forward is not None else None
        self.mixer_scale = tensors[spec.names["mixer_scale"]].float().contiguous()
        self.feed_forward_scale = None
        if feed_forward is not None:
            self.feed_forward_scale = tensors[spec.names["feed_forward_scale"]].float().contiguous()

    def input_norms(self):
        """The norms this block applies to the residual it is given."""
        return tuple(n for n in (self.mixer_norm, self.feed_forward_norm) if n is not None)

    @staticmethod
    def _normed(stream: ResidualStream, norms):
        xs = stream.take_for(norms)
        if xs is not None:
            return xs
        if all(hasattr(n, "tanh_args") for n in norms) and stream.pending is None:
            return K.tanh_norm_add(stream.h, None, None, None, None, 1.0, [n.tanh_args() for n in norms],
                                   norms[0].out_dtype)
        return [n.add_norm(stream) for n in norms]

    def forward(self, stream: ResidualStream, batch, kv, state, next_block=None) -> None:
        xs = self._normed(stream, self.input_norms())
        y1 = self.mixer.forward(xs[0], batch, kv, state)
        y2 = self.feed_forward.forward(xs[1], batch) if self.feed_forward is not None else None
        nxt = next_block.input_norms() if hasattr(next_block, "input_norms") else ()
        fused = bool(nxt) and all(hasattr(n, "tanh_args") for n in nxt)
        outs = K.tanh_norm_add(stream.h, y1, y2, self.mixer_scale, self.feed_forward_scale,
                               float(self.spec.residual_scale), [n.tanh_args() for n in nxt] if fused else [],
                               nxt[0].out_dtype if fused else torch.float32)
        stream.act = None
        stream.normed = None
        if fused:
            stream.leave_for(nxt, outs)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm)
                   if p is not None and hasattr(p, "weight_bytes")) + 4 * self.mixer_scale.numel() * \
            (2 if self.feed_forward_scale is not None else 1)


class HyperBlock:
    takes_tensors = True      # built with the checkpoint's tensors (read, write and mixing weights of the streams)
    takes_next = True         # forward gets the block that runs next

    @classmethod
    def tensor_specs(cls, spec: LayerSpec) -> List[TensorSpec]:
        S = int(spec.params.get("streams", 1))
        out = []
        for key in ("hyper1", "hyper2") if spec.feed_forward is not None else ("hyper1",):
            n = spec.names[key]
            out += [TensorSpec(n + ".in", (S,), init="ones"), TensorSpec(n + ".out", (S,), init="ones"),
                    TensorSpec(n + ".mix", (S, S))]
        return out

    def __init__(self, spec: LayerSpec, mixer, feed_forward, mixer_norm, feed_forward_norm,
                 tensors: Dict[str, torch.Tensor]):
        if spec.residual_scale != 1.0:
            raise ValueError("hyper: the write weights are the scale of a sublayer's output")
        self.spec = spec
        self.streams = int(spec.params.get("streams", 1))
        if not 1 <= self.streams <= K.hyper_max_streams():
            raise ValueError(f"hyper: {self.streams} streams (1 to {K.hyper_max_streams()})")
        self.mixer = mixer
        self.feed_forward = feed_forward              # None: the layer is its mixer only
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm if feed_forward is not None else None
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "weight"):
                raise ValueError("hyper: the sublayers' norms must be RMS norms with a weight")
        get = lambda name: tensors[name].float().contiguous()
        self.read1, self.write1, self.mix1 = (get(spec.names["hyper1"] + s) for s in (".in", ".out", ".mix"))
        self.read2 = self.write2 = self.mix2 = None
        if feed_forward is not None:
            self.read2, self.write2, self.mix2 = (get(spec.names["hyper2"] + s) for s in (".in", ".out", ".mix"))

    def first_read(self):
        """``(read weights, norm)`` of this block's first sublayer, for the block before it."""
        return self.read1, self.mixer_norm

    def _step(self, stream: ResidualStream, y, mix, write, nxt):
        """Writes ``y`` into the streams and reads for ``nxt`` = (read weights, norm) or None."""
        read, norm = nxt if nxt is not None else (None, None)
        _, r = K.hyper_step(stream.h, self.streams, y, mix, write, read, norm.weight if norm is not None else None,
                            norm.spec.eps if norm is not None else 0.0,
                            norm.out_dtype if norm is not None else torch.float32)
        return r

    def forward(self, stream: ResidualStream, batch, kv, state, next_block=None) -> None:
        S, W = self.streams, self.spec.mixer.width
        if stream.pending is not None:
            raise RuntimeError("hyper: the residual stream holds an output that was not folded in")
        left = stream.take_for((self.mixer_norm,))
        if left is not None:
            r = left[0]
        elif stream.h.shape[1] == W and S > 1:
            # the embedding's single row stands for S equal streams: the first read also widens it
            wide = torch.empty((stream.h.shape[0], S * W), dtype=torch.float32, device=stream.h.device)
            _, r = K.hyper_step(stream.h, S, None, None, None, self.read1, self.mixer_norm.weight,
                                self.mixer_norm.spec.eps, self.mixer_norm.out_dtype, out=wide)
            stream.h = wide
        else:
            r = self._step(stream, None, None, None, self.first_read())
        stream.act = None
        y = self.mixer.forward(r, batch, kv, state)
        nxt = next_block.first_read() if hasattr(next_block, "first_read") else None
        if self.feed_forward is not None:
            r = self._step(stream, y, self.mix1, self.write1, (self.read2, self.feed_forward_norm))
            y = self.feed_forward.forward(r, batch)
            r = self._step(stream, y, self.mix2, self.write2, nxt)
        else:
            r = self._step(stream, y, self.mix1, self.write1, nxt)
        stream.normed = None
        if nxt is not None:
            stream.leave_for((nxt[1],), [r])

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm)
                   if p is not None and hasattr(p, "weight_bytes"))


register_arrangement("prenorm", PreNormBlock)
register_arrangement("hyper", HyperBlock)
register_arrangement("side_by_side", SideBySideBlock)
register_arrangement("sandwich", SandwichBlock)
register_arrangement("outnorm", OutNormBlock)
