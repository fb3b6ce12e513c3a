"""Grouped-query attention with the options that newer decoders put around it.

Per token ``q, k, v = r Wq^T, r Wk^T, r Wv^T`` (one joint matrix; biases optional), ``heads`` query heads on
``kv_heads`` key/value heads (query head h reads key/value head ``h // (heads / kv_heads)``), keys and queries of
``head_dim`` features, values of ``value_dim``.  Then, each an option of the spec's ``params``:

* ``qk_norm``: ``"none"``, ``"unit"`` (each query and key head divided by its root mean square) or ``"weight"``
  (the same times a weight ``[head_dim]`` shared by all heads), with ``norm_eps``, before the rotation;
* the position encoding of the spec (``rope`` with its layout, partial rotation and stretched table, or none);
* ``v_mix``: ``"source"`` leaves this layer's values (before any mixing) for later layers of the same
  ``v_mix_key``; ``"mix"`` replaces ``v`` by ``(1 - lambda) v + lambda v_source`` with a learned scalar; the mixed
  values are what the cache keeps;
* ``sink``: one added to the softmax's denominator (a key of score 0 without a value); ``"learned"``: the sink's
  score is a learned number per query head (tensor ``sink``), neither scaled nor capped: ``exp(sink_h)`` is added;
* ``window`` of the spec > 0: a query sees the last ``window`` keys, and with ``keep_first`` > 0 also the keys at
  positions below ``keep_first`` (at their true positions);
* ``softcap`` > 0: the scaled scores become ``softcap * tanh(score / softcap)``;
* ``bias``: ``True`` (q, k, v and o have biases) or ``"qkv"`` (the output projection has none);
* ``chunk`` > 0: a query sees only the causal keys of its own block of ``chunk`` positions (counted from the
  sequence's start, however the prompt was cut);
* ``softmax_scale`` of the spec multiplies the scores.

``y = concat_h(o_h) Wo^T`` (+ bias).  Norms, rotation, mixing, scores and softmax are float32.  One kernel
(``kernels.qk_prep``) does everything between the projection and the attention and writes the cache.  In bfloat16
with keys and values of 64 or 128 features the attention is the tensor-core kernels' (tcgen05 for prompts, which
takes every option above; the TMA page stream for steps of few tokens, which takes the sink of score 0 and the blocks
but no window, cap or learned sink); everything else (float32,
other sizes, values of another width than keys) is the CUDA-core kernel in its general form
(``kernels.attn_tokens_ex``), the same for prompts, portions of prompts and single tokens.  Head sizes are padded to
a multiple of 8 in the cache (zeros), so any even size runs.

Tensor names under the mixer's prefix: ``q``, ``k``, ``v``, ``o`` (biases: the name + ``.b``), ``q.norm``,
``k.norm``, ``vmix``.

A mixer of this kind can also run on a slice of a projection that another part computed together with other
inputs' (``input_weight`` / ``forward_projected``; see ``parts/parallel.py``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .attention import BUSY_ITEMS, SPLIT_KEYS, Attention
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import position_class, register_mixer
from .spec import MixerSpec, PositionSpec

NORM_CODES = {"none": 0, "unit": 1, "weight": 2}


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class NormedAttention:
    @staticmethod
    def _sizes(spec: MixerSpec) -> Tuple[int, int, int, int]:
        dv = int(spec.params.get("value_dim", 0)) or spec.head_dim
        return spec.heads, spec.kv_heads, spec.head_dim, dv

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        H, G, d, dv = cls._sizes(spec)
        out = [TensorSpec(prefix + "q", (H * d, spec.width)), TensorSpec(prefix + "k", (G * d, spec.width)),
               TensorSpec(prefix + "v", (G * dv, spec.width)), TensorSpec(prefix + "o", (spec.width, H * dv))]
        if spec.params.get("bias", False):
            out += [TensorSpec(prefix + "q.b", (H * d,)), TensorSpec(prefix + "k.b", (G * d,)),
                    TensorSpec(prefix + "v.b", (G * dv,))]
            if spec.params["bias"] != "qkv":
                out.append(TensorSpec(prefix + "o.b", (spec.width,)))
        if spec.params.get("sink") == "learned":
            out.append(TensorSpec(prefix + "sink", (H,)))
        if spec.params.get("qk_norm", "none") == "weight":
            out += [TensorSpec(prefix + "q.norm", (d,), init="ones"), TensorSpec(prefix + "k.norm", (d,), init="ones")]
        if spec.params.get("v_mix") in ("source", "mix"):
            out.append(TensorSpec(prefix + "vmix", ()))           # the source layer stores one too and never uses it
        return out

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        H, G, d, dv = self._sizes(spec)
        if H < 1 or G < 1 or H % G != 0:
            raise ValueError(f"normed attention: {H} heads cannot share {G} kv heads")
        p = spec.params
        self.spec, self.ctx = spec, ctx
        self.H, self.G, self.d, self.dv = H, G, d, dv
        self.d_pad, self.dv_pad = pad8(d), pad8(dv)
        self.norm = NORM_CODES[p.get("qk_norm", "none")]
        self.eps = float(p.get("norm_eps", 1e-6))
        self.sink = bool(p.get("sink", False))
        self.sink_vals = tensors[prefix + "sink"].float().contiguous() if p.get("sink") == "learned" else None
        self.chunk = int(p.get("chunk", 0))
        self.window = int(spec.window)
        self.keep_first = int(p.get("keep_first", 0)) if self.window > 0 else 0
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        if self.window < 0 or self.keep_first < 0 or self.softcap < 0:
            raise ValueError("normed attention: window, keep_first and softcap must not be negative")
        self.v_mix = p.get("v_mix")
        self.v_mix_key = ("v_mix", p.get("v_mix_key", 0))
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else d ** -0.5
        bias = bool(p.get("bias", False))
        self._w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("q", "k", "v")], dim=0)
        self._b = torch.cat([tensors[prefix + n + ".b"].to(ctx.dtype) for n in ("q", "k", "v")]) if bias else None
        self.n_proj = self._w.shape[0]
        self.qkv: Optional[Linear] = None                   # made on first use: a parallel part may project for us
        wo = tensors[prefix + "o"].to(ctx.dtype)
        if self.dv_pad != dv:                               # the attention's rows are padded: zero columns for the pad
            wo = torch.nn.functional.pad(wo.view(spec.width, H, dv), (0, self.dv_pad - dv)).reshape(spec.width, -1)
        self.o = Linear(wo, tensors[prefix + "o.b"] if bias and p["bias"] != "qkv" else None, ctx.dtype)
        self.q_w = tensors[prefix + "q.norm"].float().contiguous() if self.norm == 2 else None
        self.k_w = tensors[prefix + "k.norm"].float().contiguous() if self.norm == 2 else None
        self.lam = tensors[prefix + "vmix"].float().reshape(1).contiguous() if self.v_mix == "mix" else None
        pos = spec.position or PositionSpec(kind="none", dims=0)
        self.position = position_class(pos.kind)(pos, d, ctx)
        self.rot = int(self.position.spec.dims)
        # How the tensor-core kernels cut a step's work is the attention part's business: a block of ``chunk``
        # positions bounds a query's keys as a window of that many keys does.
        self._cuts = Attention.__new__(Attention)
        self._cuts.spec = MixerSpec(kind="attention", width=spec.width, heads=H, kv_heads=G, head_dim=self.d_pad,
                                    window=self.chunk or (self.window + self.keep_first if self.window else 0))
        # what the tensor-core kernels do not apply
        self._plain_scores = self.window == 0 and self.softcap == 0.0 and self.sink_vals is None

    # -- what a part that projects for several mixers at once needs -----------------------------------------------
    def input_weight(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        return self._w, self._b

    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(self.G, self.d_pad, self.window, self.dv_pad if self.dv_pad != self.d_pad else 0, chunk=self.chunk,
                         keep_first=self.keep_first)

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if self.qkv is None:
            self.qkv = Linear(self._w, self._b, self.ctx.dtype)
        proj = self.qkv(x, out_dtype=self.qkv.wide_dtype(x.shape[0]))
        return self.forward_projected(proj, 0, batch, kv, state)

    def forward_projected(self, proj: torch.Tensor, off: int, batch, kv, state) -> torch.Tensor:
        """``proj [T, *]`` holds this mixer's ``[q | k | v]`` from column ``off`` on."""
        if kv is None or not kv.owns:
            raise RuntimeError("normed attention needs a cache view of its own")
        H, G, d, dv = self.H, self.G, self.d, self.dv
        T = proj.shape[0]
        q_off, k_off, v_off = off, off + H * d, off + (H + G) * d
        mix = None
        if self.v_mix == "source":
            batch.memo[self.v_mix_key] = proj[:, v_off:v_off + G * dv]
        elif self.v_mix == "mix":
            src = batch.memo.get(self.v_mix_key)
            if src is None:
                raise RuntimeError("normed attention: no earlier layer left its values to mix in")
            mix = (self.lam, src)
        q, _ = K.qk_prep(proj, q_off, k_off, v_off, H, G, d, dv, self.d_pad, self.dv_pad, self.norm, self.q_w, self.k_w,
                         self.eps, self.rot, self.position.layout_code, self.position.table if self.rot else None,
                         self.position.mscale, 1.0, mix, batch.tok_pos, batch.tok_seq, kv.block_table, kv.page_size,
                         self.ctx.dtype, kv.k, kv.v)
        out = torch.empty((T, H * self.dv_pad), dtype=self.ctx.dtype, device=proj.device)
        if self._tensor_cores(q, out, batch, kv):
            return self.o(out, out_dtype=self.o.wide_dtype(T))
        split = max(SPLIT_KEYS, kv.page_size)
        if split % kv.page_size:
            split = kv.page_size * (split // kv.page_size + 1)
        n = self._chunks(batch.max_kv_len, split)
        # bfloat16 with more work items than the GPU holds at once: chunks twice as long (float32 keeps one chunking
        # for every batch, so that its results do not depend on the batch at all)
        if self.ctx.dtype == torch.bfloat16 and T * G * n > BUSY_ITEMS:
            split *= 2
            n = self._chunks(batch.max_kv_len, split)
        scratch = None
        if n > 1:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, H, self.dv_pad, n) // 4)
        K.attn_tokens_ex(q, q.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T, H, G,
                         self.d_pad, self.dv_pad, kv.page_size, self.window, self.chunk, self.sink, self.scale, split, n,
                         scratch, keep_first=self.keep_first, softcap=self.softcap, sink_vals=self.sink_vals)
        return self.o(out, out_dtype=self.o.wide_dtype(T))

    def _tensor_cores(self, q: torch.Tensor, out: torch.Tensor, batch, kv) -> bool:
        """bfloat16 with keys and values of 64 or 128 features: prompts through the tcgen05 kernel, steps of few
        tokens through the kernel that streams pages by TMA, both with the sink and the blocks of positions as
        parameters.  False when the sizes are not theirs (the CUDA-core kernel then takes the step)."""
        if self.ctx.dtype != torch.bfloat16 or self.d_pad != self.dv_pad or self.d_pad != self.d:
            return False
        H, G, d, T = self.H, self.G, self.d, q.shape[0]
        if batch.max_new > 1 and batch.tiles and K.attn_prefill_tc_supported(torch.bfloat16, d, kv.page_size):
            tile_seq, tile_q0, n_tiles = batch.tiles[128]
            key = ("attn_prefill_variant", H, d, self.chunk, self.window, self.keep_first)
            variant = batch.memo.get(key)
            if variant is None:
                variant = batch.memo[key] = self._cuts._prefill_variant(batch.tile_keys.get(128), kv.page_size, q.device)
            K.attn_prefill_tc(q, q.stride(0), out, kv.k, kv.v, kv.block_table, batch.row_start, batch.row_pos0, tile_seq,
                              tile_q0, n_tiles, H, G, d, kv.page_size, self.window, self.scale, variant=variant,
                              chunk=self.chunk, sink=self.sink, keep_first=self.keep_first, softcap=self.softcap,
                              sink_vals=self.sink_vals)
            return True
        if not self._plain_scores:
            return False                 # single tokens with a window, a cap or sink scores: the CUDA-core kernel
        if not K.attn_decode_supported(torch.bfloat16, T, H, G, d, kv.page_size, kv.page_size, 1):
            return False
        split, head_split, in_block = self._cuts._decode_split(T, batch.max_kv_len, kv.page_size, q.device)
        head_split, twins = self._cuts._decode_twins(head_split, in_block)
        n = self._cuts._chunks(batch.max_kv_len, split)
        scratch = None
        if n > 1 and not in_block:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, H, d, n) // 4)
        K.attn_decode(q, q.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T, H, G, d,
                      kv.page_size, 0, self.scale, split, n, scratch, head_split=head_split, in_block=in_block,
                      twins=twins, chunk=self.chunk, sink=self.sink)
        return True

    def _chunks(self, max_kv_len: int, split: int) -> int:
        """The most pieces of ``split`` keys that a token's visible keys can touch."""
        n = (max_kv_len + split - 1) // split
        if self.chunk > 0:
            n = min(n, (self.chunk + split - 2) // split + 1)
        if self.window > 0:
            # the pieces a window can touch, and those of the kept first keys before them
            n = min(n, (self.window + split - 2) // split + 1 + (self.keep_first + split - 1) // split)
        return max(1, n)

    def weight_bytes(self) -> int:
        n = self._w.numel() * self._w.element_size() + self.o.weight_bytes()
        if self._b is not None:
            n += self._b.numel() * self._b.element_size()
        return n


register_mixer("normed_attention", NormedAttention)
