"""Token embedding and output head.

Embedding: ``h0[t] = E[id_t] * scale`` (the gather is src/model.cpp:529; the
scale is MiniCPM's ``scale_emb``).  Head: ``logits = (norm(h) / divisor) W^T``
in float32, computed only for the rows that were asked for (the reference
computes every row, src/model.cpp:589-592); ``W`` is the embedding table when
the head is tied.  With ``softcap`` c > 0 in the head's parameters the logits become ``c tanh(logits / c)``.

Both are registered part kinds like the others (``"table"`` and ``"linear"``).  An embedding of another kind has
``tensor_specs(spec)``, ``__init__(spec, tensors, ctx)`` and ``forward(token_ids) -> ResidualStream``; a head has
``tensor_specs(spec)``, ``__init__(spec, tensors, embedding, ctx)``, ``forward(stream, final_norm, rows) ->
float32 logits [rows, vocab]`` and ``read_bytes()``, the weight bytes a step reads.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, ResidualStream, StateRequest
from .linear import Linear
from .registry import register_embedding, register_head
from .spec import EmbeddingSpec, HeadSpec


class Embedding:
    @staticmethod
    def tensor_specs(spec: EmbeddingSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.name, (spec.vocab, spec.width))]

    def __init__(self, spec: EmbeddingSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec = spec
        self.table = tensors[spec.name].to(ctx.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor) -> ResidualStream:
        return ResidualStream(K.embed(token_ids, self.table, float(self.spec.scale)))

    def weight_bytes(self) -> int:
        return self.table.numel() * self.table.element_size()


class Head:
    @staticmethod
    def tensor_specs(spec: HeadSpec) -> List[TensorSpec]:
        if spec.tied:
            return []
        # tied None: the configuration does not say; a head of its own is used when the checkpoint has one
        return [TensorSpec(spec.name, (spec.vocab, spec.width), optional=spec.tied is None)]

    def __init__(self, spec: HeadSpec, tensors: Dict[str, torch.Tensor], embedding: Embedding, ctx: BuildContext):
        self.spec = spec
        self.tied = spec.tied if spec.tied is not None else spec.name not in tensors
        weight = embedding.table if self.tied else tensors[spec.name]
        self.linear = Linear(weight, None, ctx.dtype)
        if self.tied:
            self.linear.weight = embedding.table          # one copy in memory

    def forward(self, stream: ResidualStream, final_norm, rows: Optional[torch.Tensor]) -> torch.Tensor:
        r = final_norm.add_norm(stream, rows=rows, out_scale=1.0 / float(self.spec.input_divisor))
        logits = self.linear(r, out_dtype=torch.float32)
        cap = float(self.spec.params.get("softcap", 0.0))
        if cap > 0.0:
            K.softcap(logits, cap)              # logits <- cap * tanh(logits / cap)
        return logits

    def weight_bytes(self) -> int:
        """Bytes this part holds beyond the embedding's."""
        return 0 if self.tied else self.linear.weight_bytes()

    def read_bytes(self) -> int:
        """Weight bytes a step reads for the logits (a tied head reads the embedding table)."""
        return self.linear.weight_bytes()


class HashedPairEmbedding:
    """``h0[t] = E[id_t] + P[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]``: the token's row plus a row of a
    second table picked by a hash of the token and the one before it; a sequence's first token takes the second
    table's last row (number ``buckets``).  The token before a step's first token is per-sequence state (an int32
    per slot) that the kernel keeps up.  Parameters of the spec: ``pair_name``, ``buckets``, ``mul_prev``,
    ``mul_cur``."""

    takes_batch = True

    @staticmethod
    def tensor_specs(spec: EmbeddingSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.name, (spec.vocab, spec.width)),
                TensorSpec(spec.params["pair_name"], (int(spec.params["buckets"]) + 1, spec.width))]

    def __init__(self, spec: EmbeddingSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if float(spec.scale) != 1.0:
            raise ValueError("hashed pair embedding: no scale on the sum of two rows")
        self.spec = spec
        self.table = tensors[spec.name].to(ctx.dtype).contiguous()
        self.pairs = tensors[spec.params["pair_name"]].to(ctx.dtype).contiguous()
        self.buckets = int(spec.params["buckets"])
        self.mul_prev, self.mul_cur = int(spec.params["mul_prev"]), int(spec.params["mul_cur"])

    def state_request(self) -> StateRequest:
        return StateRequest((), torch.int32)

    def forward(self, token_ids: torch.Tensor, batch, state: Optional[torch.Tensor]) -> ResidualStream:
        if state is None:
            raise RuntimeError("the hashed pair embedding needs its per-sequence state")
        return ResidualStream(K.embed_hashed(token_ids, batch.tok_pos, batch.tok_seq, batch.row_start, batch.slot_ids,
                                             self.table, self.pairs, self.buckets, self.mul_prev, self.mul_cur, state))

    def weight_bytes(self) -> int:
        return (self.table.numel() + self.pairs.numel()) * self.table.element_size()


register_embedding("table", Embedding)
register_embedding("table_hashed_pair", HashedPairEmbedding)
register_head("linear", Head)
