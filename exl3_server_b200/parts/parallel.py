"""A mixer made of two mixers side by side that read the same input.

``y = coef * (rmsnorm(a(r)) * wa + rmsnorm(b(r)) * wb)``: each branch's output is normed over the model width with
a weight of its own (a plain factor, ``norm_eps``), and the two are summed with one constant (1/2: their mean).
The branches are any registered mixers (``params["branches"]``: two ``MixerSpec``; ``params["prefixes"]``: their
tensor-name prefixes under this mixer's; ``params["out_names"]``: the names of the two norm weights).  At most one
branch may ask for keys and values and at most one for per-sequence state: a schedule entry has one of each.

With ``params["combine"] = "weighted"`` the branches' outputs are not normed: ``y = sa * a(r) + sb * b(r)`` with the
two constants ``params["scales"]`` (one float32 kernel, ``kernels.scaled_sum2``; no ``out_names`` then).

When both branches can run on a slice of a projection (``input_weight`` / ``forward_projected``), their input
matrices are one matrix and the step reads ``r`` once.  The norms and the sum are one float32 kernel
(``kernels.normed_sum2``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest
from .linear import Linear
from .registry import mixer_class, register_mixer
from .spec import MixerSpec


class ParallelMixer:
    @staticmethod
    def _parts(spec: MixerSpec):
        branches, prefixes = spec.params["branches"], spec.params["prefixes"]
        weighted = spec.params.get("combine", "normed_mean") == "weighted"
        outs = [] if weighted else spec.params["out_names"]
        if len(branches) != 2 or len(prefixes) != 2 or len(outs) != (0 if weighted else 2):
            raise ValueError("parallel mixer: two branches, two prefixes and two output-norm names")
        if weighted and len(spec.params.get("scales", ())) != 2:
            raise ValueError("parallel mixer: a weighted sum needs two scales")
        return branches, prefixes, outs

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        branches, prefixes, outs = cls._parts(spec)
        specs: List[TensorSpec] = []
        for b, p in zip(branches, prefixes):
            specs += mixer_class(b.kind).tensor_specs(b, prefix + p)
        return specs + [TensorSpec(prefix + n, (spec.width,), init="ones") for n in outs]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        branches, prefixes, outs = self._parts(spec)
        self.spec, self.ctx = spec, ctx
        self.coef = float(spec.params.get("coef", 0.5))
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        self.a, self.b = (mixer_class(b.kind)(b, tensors, prefix + p, ctx) for b, p in zip(branches, prefixes))
        self.scales = tuple(float(s) for s in spec.params["scales"]) if not outs else None
        if outs:
            self.wa, self.wb = (tensors[prefix + n].float().contiguous() for n in outs)
        if sum(m.cache_request() is not None for m in (self.a, self.b)) > 1 or \
                sum(m.state_request() is not None for m in (self.a, self.b)) > 1:
            raise ValueError("parallel mixer: at most one branch with keys and values and one with state")
        self.joint: Optional[Linear] = None
        if all(hasattr(m, "input_weight") and hasattr(m, "forward_projected") for m in (self.a, self.b)):
            (wa, ba), (wb, bb) = self.a.input_weight(), self.b.input_weight()
            bias = None
            if ba is not None or bb is not None:
                zeros = lambda w: torch.zeros(w.shape[0], dtype=ctx.dtype, device=w.device)
                bias = torch.cat([ba if ba is not None else zeros(wa), bb if bb is not None else zeros(wb)])
            self.joint = Linear(torch.cat([wa, wb], dim=0), bias, ctx.dtype)
            self.split = wa.shape[0]
            # one copy in memory: the branches' own matrices become views of the joint one
            self.a._w, self.b._w = self.joint.weight[:self.split], self.joint.weight[self.split:]

    def cache_request(self) -> Optional[KVRequest]:
        return self.a.cache_request() or self.b.cache_request()

    def state_request(self):
        return self.a.state_request() or self.b.state_request()

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if self.joint is not None:
            proj = self.joint(x, out_dtype=self.joint.wide_dtype(x.shape[0]))
            # a branch that also reads the input itself (low-rank side projections) says so
            extra = lambda m: {"x": x} if getattr(m, "wants_input", False) else {}
            ya = self.a.forward_projected(proj, 0, batch, kv, state, **extra(self.a))
            yb = self.b.forward_projected(proj, self.split, batch, kv, state, **extra(self.b))
        else:
            ya = self.a.forward(x, batch, kv, state)
            yb = self.b.forward(x, batch, kv, state)
        if self.scales is not None:
            if ya.dtype != yb.dtype:
                ya, yb = ya.float(), yb.float()
            return K.scaled_sum2(ya, yb, self.scales[0], self.scales[1])
        return K.normed_sum2(ya, yb, self.wa, self.wb, self.eps, self.coef)

    def weight_bytes(self) -> int:
        return self.a.weight_bytes() + self.b.weight_bytes()


register_mixer("parallel", ParallelMixer)
