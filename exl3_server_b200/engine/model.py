"""A model assembled from a plan: embedding, layers built from registered
parts, the schedule that orders them, the final norm and the head.

The forward pass runs exactly the tokens of a ``StepBatch`` against the cache
and returns float32 logits for the wanted rows.  It is the reference's
``Model::forward_multi`` (src/model.cpp:514-628) for a packed batch of
sequences with a paged cache.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.kv import SequenceCache
from ..parts.base import BuildContext, KVRequest, StateRequest
from ..parts.registry import (arrangement_class, embedding_class, feed_forward_class, head_class, mixer_class,
                              norm_class)
from ..parts.spec import ModelPlan
from ..weights.loader import TensorSpec
from .batch import StepBatch


def plan_manifest(plan: ModelPlan) -> List[TensorSpec]:
    """Every tensor the plan's parts will ask for, by checkpoint name."""
    specs: List[TensorSpec] = list(embedding_class(plan.embedding.kind).tensor_specs(plan.embedding))
    for layer in plan.layers:
        specs += mixer_class(layer.mixer.kind).tensor_specs(layer.mixer, layer.names["mixer"])
        specs += norm_class(layer.mixer_norm.kind).tensor_specs(layer.mixer_norm, layer.names["mixer_norm"])
        if layer.mixer_out_norm is not None:
            specs += norm_class(layer.mixer_out_norm.kind).tensor_specs(layer.mixer_out_norm,
                                                                        layer.names["mixer_out_norm"])
        if layer.feed_forward is not None and layer.feed_forward_out_norm is not None:
            specs += norm_class(layer.feed_forward_out_norm.kind).tensor_specs(layer.feed_forward_out_norm,
                                                                               layer.names["feed_forward_out_norm"])
        if layer.feed_forward is not None:
            specs += feed_forward_class(layer.feed_forward.kind).tensor_specs(layer.feed_forward,
                                                                             layer.names["feed_forward"])
            specs += norm_class(layer.feed_forward_norm.kind).tensor_specs(layer.feed_forward_norm,
                                                                          layer.names["feed_forward_norm"])
    for layer in plan.layers:
        arrangement = arrangement_class(layer.arrangement)
        if hasattr(arrangement, "tensor_specs"):            # arrangements with tensors of their own (layer scales)
            specs += arrangement.tensor_specs(layer)
    specs += norm_class(plan.final_norm.kind).tensor_specs(plan.final_norm, plan.final_norm_name)
    specs += head_class(plan.head.kind).tensor_specs(plan.head)
    return specs


class Model:
    def __init__(self, plan: ModelPlan, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        ctx = BuildContext(dtype=dtype, device=self.device)
        self.embedding = embedding_class(plan.embedding.kind)(plan.embedding, tensors, ctx)
        self.blocks = []
        for layer in plan.layers:
            mixer = mixer_class(layer.mixer.kind)(layer.mixer, tensors, layer.names["mixer"], ctx)
            n1 = norm_class(layer.mixer_norm.kind)(layer.mixer_norm, tensors, layer.names["mixer_norm"], ctx)
            ff = n2 = None
            if layer.feed_forward is not None:
                ff = feed_forward_class(layer.feed_forward.kind)(layer.feed_forward, tensors,
                                                                 layer.names["feed_forward"], ctx)
                n2 = norm_class(layer.feed_forward_norm.kind)(layer.feed_forward_norm, tensors,
                                                              layer.names["feed_forward_norm"], ctx)
            if layer.mixer_out_norm is not None or layer.feed_forward_out_norm is not None:
                outs = [None, None]
                if layer.mixer_out_norm is not None:
                    outs[0] = norm_class(layer.mixer_out_norm.kind)(layer.mixer_out_norm, tensors,
                                                                    layer.names["mixer_out_norm"], ctx)
                if ff is not None and layer.feed_forward_out_norm is not None:
                    outs[1] = norm_class(layer.feed_forward_out_norm.kind)(layer.feed_forward_out_norm, tensors,
                                                                           layer.names["feed_forward_out_norm"], ctx)
                self.blocks.append(arrangement_class(layer.arrangement)(layer, mixer, ff, n1, n2, out_norms=tuple(outs)))
            elif getattr(arrangement_class(layer.arrangement), "takes_tensors", False):
                self.blocks.append(arrangement_class(layer.arrangement)(layer, mixer, ff, n1, n2, tensors=tensors))
            else:
                self.blocks.append(arrangement_class(layer.arrangement)(layer, mixer, ff, n1, n2))
        self.final_norm = norm_class(plan.final_norm.kind)(plan.final_norm, tensors, plan.final_norm_name, ctx)
        self.head = head_class(plan.head.kind)(plan.head, tensors, self.embedding, ctx)
        self.vocab = plan.head.vocab

    def cache_requests(self) -> List[Tuple[Optional[KVRequest], Optional[StateRequest], Optional[int]]]:
        out = []
        for e in self.plan.schedule:
            m = self.blocks[e.layer].mixer
            out.append((m.cache_request(), m.state_request(), e.cache_from))
        return out

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> SequenceCache:
        extra = {}
        if getattr(self.embedding, "state_request", None) is not None:
            req = self.embedding.state_request()
            if req is not None:
                extra["embedding"] = req
        return SequenceCache(self.cache_requests(), max_tokens, dtype=self.dtype, device=self.device,
                             max_slots=max_slots, extra_states=extra)

    def forward(self, batch: StepBatch, cache: SequenceCache) -> Optional[torch.Tensor]:
        if getattr(self.embedding, "takes_batch", False):
            # an embedding that looks beyond the token itself (the token before, positions) gets the step and its
            # per-sequence state
            stream = self.embedding.forward(batch.token_ids, batch, cache.state_of("embedding"))
        else:
            stream = self.embedding.forward(batch.token_ids)
        sched = self.plan.schedule
        for i, e in enumerate(sched):
            block = self.blocks[e.layer]
            kv, state = cache.view(i, batch.block_tables), cache.state_of(i)
            if getattr(block, "takes_next", False):
                # the block that runs next, so that this block's last kernel may also apply that block's first norms
                block.forward(stream, batch, kv, state,
                              next_block=self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None)
            elif getattr(block, "takes_after", False):
                # the norm that the next block applies first, so that this block's last projection may apply it
                nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
                block.forward(stream, batch, kv, state, after=getattr(nxt, "mixer_norm", None))
            else:
                block.forward(stream, batch, kv, state)
        if batch.n_wanted == 0:
            return None
        return self.head.forward(stream, self.final_norm, batch.want_rows)

    def weight_bytes(self, tokens: Optional[int] = None) -> int:
        """Bytes of weights that one step reads (each matrix once; a tied head
        reads the embedding table).  With ``tokens``, routed feed-forwards count the
        experts that a step of so many tokens is expected to pick; without, all."""
        n = sum(self.blocks[e.layer].weight_bytes() for e in self.plan.schedule)
        if tokens is not None:
            for e in self.plan.schedule:
                ff = getattr(self.blocks[e.layer], "feed_forward", None)
                if hasattr(ff, "untouched_bytes"):
                    n -= ff.untouched_bytes(tokens)
        n += self.final_norm.weight_bytes()
        n += self.head.read_bytes()
        return n
