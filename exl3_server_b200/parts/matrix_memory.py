"""Mixers whose matrix state is updated by more than a decayed sum (``csrc/matrix_memory.cu``).

``mlstm``: a matrix memory with exponential gates.  ``q = Wq r * dk^(-1/2)``, ``k = Wk r`` (``heads x dk``), ``v = Wv r``
(``heads x dv``); per head a log input gate ``i = cap tanh((Wi r + bi) / cap)`` and a log forget gate
``f = logsigmoid(cap tanh((Wf r + bf) / cap))``; a running maximum ``m`` that starts at 0 keeps the exponentials in
range: ``m' = max(f + m, i)``, ``S' = exp(f + m - m') S + exp(i - m') k v^T``, ``n'`` the same with ``k`` alone,
``o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)``.  Each head's ``o`` is divided by its root mean square, the heads
are concatenated, multiplied by a weight and by ``sigmoid(Wg r)``, and projected by ``Wo``.  Parameters: ``key_dim``,
``value_dim``, ``gate_cap``, ``norm_eps``.  Tensors: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``i``, ``i.b``,
``f``, ``f.b``.  State per sequence: ``S`` (kept column by column, ``[heads, dv, dk]``), ``n [heads, dk]``, ``m [heads]``.

``gated_delta``: the gated delta rule.  ``q = Wq r``, ``k = Wk r`` (``qk_heads x dk``), ``v = Wv r`` (``heads x dv``;
value head h reads q/k head ``h // (heads / qk_heads)``); each passes a short causal convolution over time per channel
(``taps`` taps, the last one the current token's, no bias, zeros before the start) and SiLU; q and k heads become
unit vectors (``x / sqrt(sum x^2 + unit_eps)``), q times ``dk^(-1/2)``.  ``beta = sigmoid(Wb r)`` per head; a decay per
head and key channel ``g = exp(-exp(A_h) softplus(Wa2 (Wa1 r) + dt_bias))``.  Per head ``S <- diag(g) S``,
``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q`` (the read sees the token's own write).  Each head's ``o``
is divided by its root mean square, times a weight ``[dv]`` shared by the heads, times ``sigmoid(Wg2 (Wg1 r))``, then
``Wo``.  Parameters: ``qk_heads``, ``key_dim``, ``value_dim``, ``taps``, ``norm_eps``, ``unit_eps``; the ranks of the two
low-rank pairs are whatever the checkpoint has.  Tensors: ``q``, ``q.conv``, ``k``, ``k.conv``, ``v``, ``v.conv``,
``b``, ``A_log``, ``norm``, ``a1``, ``a2``, ``dt_bias``, ``g1``, ``g2``, ``o``.  State per sequence: every channel's last
``taps - 1`` inputs of the convolution, and ``S`` (kept column by column, ``[heads, dv, dk]``).

Gates, decays with their exponentials and softplus, unit norms, the states and the per-head norms are float32; the
projections are the model's type (float32 results where the projection's kernel has them for free).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import register_mixer
from .spec import MixerSpec


class MLSTM:
    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int]:
        dk = int(spec.params["key_dim"])
        return spec.heads, dk, int(spec.params.get("value_dim", 0)) or dk

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, dk, dv = cls._sizes(spec)
        W = spec.width
        return [TensorSpec(prefix + "q", (H * dk, W)), TensorSpec(prefix + "k", (H * dk, W)),
                TensorSpec(prefix + "v", (H * dv, W)), TensorSpec(prefix + "g", (H * dv, W)),
                TensorSpec(prefix + "o", (W, H * dv)), TensorSpec(prefix + "norm", (H * dv,), init="ones"),
                TensorSpec(prefix + "i", (H, W)), TensorSpec(prefix + "i.b", (H,)),
                TensorSpec(prefix + "f", (H, W)), TensorSpec(prefix + "f.b", (H,))]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, dk, dv = self._sizes(spec)
        self.cap = float(spec.params["gate_cap"])
        if H < 1 or dk < 1 or dv < 1 or not self.cap > 0:
            raise ValueError("mlstm: heads, key_dim, value_dim and gate_cap must be positive")
        self.spec, self.ctx = spec, ctx
        self.H, self.dk, self.dv = H, dk, dv
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        # one matrix [q | k | v | g | i | f] with the gates' biases: steps of few tokens get float32 results from one
        # projection; steps of many get 16-bit q, k, v, g from its first rows and the two gates' pre-activations, which
        # stay float32 whatever the step's size, from a product of their own over its last rows
        n_main = 2 * H * dk + 2 * H * dv
        w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("q", "k", "v", "g", "i", "f")], dim=0)
        b = torch.cat([torch.zeros(n_main, dtype=ctx.dtype, device=w.device), tensors[prefix + "i.b"].to(ctx.dtype),
                       tensors[prefix + "f.b"].to(ctx.dtype)])
        self.joint = Linear(w, b, ctx.dtype)
        self.proj = Linear(self.joint.weight[:n_main], None, ctx.dtype)            # views: one copy in memory
        self.gates = Linear(self.joint.weight[n_main:], self.joint.bias[n_main:], ctx.dtype)
        self.n_main = n_main
        self.norm_w = tensors[prefix + "norm"].float().contiguous()
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self):
        return (StateRequest((self.H, self.dv, self.dk), torch.float32), StateRequest((self.H, self.dk), torch.float32),
                StateRequest((self.H,), torch.float32))

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if state is None:
            raise RuntimeError("mlstm needs its per-sequence state")
        S, n, m = state
        H, dk, dv = self.H, self.dk, self.dv
        T = x.shape[0]
        if self.joint.wide_dtype(T) == torch.float32:
            proj = self.joint(x, out_dtype=torch.float32)
            z = proj[:, self.n_main:]
        else:
            proj = self.proj(x, out_dtype=self.ctx.dtype)
            if x.shape[1] % 8 == 0:
                # a handful of output features for many rows: a warp a row, float32 results in one launch
                z = K.gemm_few_out(x, self.gates.weight, self.gates.bias)
            else:
                z = self.gates(x, out_dtype=torch.float32)
        q, k = proj[:, :H * dk], proj[:, H * dk:2 * H * dk]
        v = proj[:, 2 * H * dk:2 * H * dk + H * dv]
        g = proj[:, 2 * H * dk + H * dv:]
        need = K.mlstm_scan_scratch_bytes(batch.n_rows, T, H, dk, dv, batch.max_new)
        o = K.mlstm_scan(q, k, v, z[:, :H], z[:, H:], self.cap, float(dk) ** -0.5, S, n, m, batch.slot_ids,
                         batch.row_start, batch.n_rows, H, dk, dv, batch.max_new,
                         scratch=batch.workspace.plain(need // 4) if need else None)
        y = K.head_norm_gate(o, self.norm_w, g, self.eps, H, dv, self.ctx.dtype, gate_kind="sigmoid")
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self.joint.weight_bytes() + self.o.weight_bytes() + 4 * self.norm_w.numel()


class GatedDelta:
    wants_input = True        # ``forward_projected`` also takes the mixer's input (for the low-rank pairs)

    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int, int, int]:
        dk = int(spec.params["key_dim"])
        G = int(spec.params.get("qk_heads", 0)) or spec.heads
        return spec.heads, G, dk, int(spec.params.get("value_dim", 0)) or dk, int(spec.params.get("taps", 4))

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, G, dk, dv, taps = cls._sizes(spec)
        W = spec.width
        free = 16
        return [TensorSpec(prefix + "q", (G * dk, W)), TensorSpec(prefix + "q.conv", (G * dk, taps)),
                TensorSpec(prefix + "k", (G * dk, W)), TensorSpec(prefix + "k.conv", (G * dk, taps)),
                TensorSpec(prefix + "v", (H * dv, W)), TensorSpec(prefix + "v.conv", (H * dv, taps)),
                TensorSpec(prefix + "b", (H, W)), TensorSpec(prefix + "A_log", (H,)),
                TensorSpec(prefix + "norm", (dv,), init="ones"),
                TensorSpec(prefix + "a1", (-1, W), free_dim=free), TensorSpec(prefix + "a2", (H * dk, -1), free_dim=free),
                TensorSpec(prefix + "dt_bias", (H * dk,)),
                TensorSpec(prefix + "g1", (-1, W), free_dim=free), TensorSpec(prefix + "g2", (H * dv, -1), free_dim=free),
                TensorSpec(prefix + "o", (W, H * dv))]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, G, dk, dv, taps = self._sizes(spec)
        if H < 1 or G < 1 or H % G != 0 or dk < 1 or dv < 1:
            raise ValueError(f"gated delta: {H} value heads cannot share {G} query/key heads")
        if not 1 <= taps <= K.conv_prep_max_taps():
            raise ValueError(f"gated delta: {taps} taps (at most {K.conv_prep_max_taps()})")
        self.spec, self.ctx = spec, ctx
        self.H, self.G, self.dk, self.dv, self.taps = H, G, dk, dv, taps
        self.eps = float(spec.params.get("norm_eps", 1e-6))
        self.unit_eps = float(spec.params.get("unit_eps", 1e-6))
        self._w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("q", "k", "v", "b")], dim=0)
        self.n_proj = self._w.shape[0]
        self.proj: Optional[Linear] = None                  # made on first use: a parallel part may project for us
        self.conv = [tensors[prefix + n + ".conv"].float().contiguous() for n in ("q", "k", "v")]
        a1, a2, g1, g2 = (tensors[prefix + n].to(ctx.dtype) for n in ("a1", "a2", "g1", "g2"))
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ValueError(f"gated delta: {prefix}a1/a2 or {prefix}g1/g2 disagree about their rank")
        ra, rg = a1.shape[0], g1.shape[0]
        # both low-rank pairs as two projections: [a1; g1], then a block-diagonal [a2 0; 0 g2]
        self.low = Linear(torch.cat([a1, g1], dim=0), None, ctx.dtype)
        second = torch.zeros((H * dk + H * dv, ra + rg), dtype=ctx.dtype, device=a2.device)
        second[:H * dk, :ra] = a2
        second[H * dk:, ra:] = g2
        self.second = Linear(second, None, ctx.dtype)
        self.a_log = tensors[prefix + "A_log"].float().contiguous()
        self.dt_bias = tensors[prefix + "dt_bias"].float().contiguous()
        self.norm_w = tensors[prefix + "norm"].float().repeat(H).contiguous()          # one weight for every head
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def input_weight(self):
        return self._w, None

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self):
        channels = 2 * self.G * self.dk + self.H * self.dv
        return (StateRequest((channels, self.taps - 1), torch.float32),
                StateRequest((self.H, self.dv, self.dk), torch.float32))

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if self.proj is None:
            self.proj = Linear(self._w, None, self.ctx.dtype)
        proj = self.proj(x, out_dtype=self.proj.wide_dtype(x.shape[0]))
        return self.forward_projected(proj, 0, batch, kv, state, x=x)

    def forward_projected(self, proj: torch.Tensor, off: int, batch, kv, state, x=None) -> torch.Tensor:
        """``proj [T, *]`` holds this mixer's ``[q | k | v | b]`` from column ``off`` on; ``x`` is the mixer's input."""
        if state is None or x is None:
            raise RuntimeError("gated delta needs its per-sequence state and the mixer's input")
        conv_state, S = state
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        T = proj.shape[0]
        k_off, v_off, b_off = off + G * dk, off + 2 * G * dk, off + 2 * G * dk + H * dv
        qkv = K.conv_prep(proj, off, k_off, v_off, self.conv[0], self.conv[1], self.conv[2], G, dk, H, dv,
                          self.unit_eps, float(dk) ** -0.5, conv_state, batch.slot_ids, batch.row_start, batch.n_rows,
                          batch.max_new)
        low = self.low(x, out_dtype=self.ctx.dtype)
        z = self.second(low, out_dtype=self.second.wide_dtype(T))
        need = K.delta_scan_scratch_bytes(batch.n_rows, T, H, dk, dv, batch.max_new)
        o = K.delta_scan(qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], proj[:, b_off:b_off + H],
                         z[:, :H * dk], self.a_log, self.dt_bias, S, batch.slot_ids, batch.row_start, batch.n_rows,
                         H, G, dk, dv, batch.max_new, scratch=batch.workspace.plain(need // 4) if need else None)
        y = K.head_norm_gate(o, self.norm_w, z[:, H * dk:], self.eps, H, dv, self.ctx.dtype, gate_kind="sigmoid")
        return self.o(y, out_dtype=self.o.wide_dtype(T))

    def weight_bytes(self) -> int:
        return self._w.numel() * self._w.element_size() + self.low.weight_bytes() + self.second.weight_bytes() + \
            self.o.weight_bytes()


register_mixer("mlstm", MLSTM)
register_mixer("gated_delta", GatedDelta)
