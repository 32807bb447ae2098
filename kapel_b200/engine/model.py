"""A model as built parts, and its forward pass over one step's rows.

The order of layers is the spec's `schedule`: a list of (layer, whose cache), so a layer may
run twice or read another layer's keys and values; a run may have a cache of its own (`replica`)
and a part that rewrites the stream ahead of it (`before`). Kapel's forward pass is
crates/kapel-models/src/model.rs:1272-1383: embed, blocks, the rows wanted, final norm, head.
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from .. import kernels as K
from ..cache import CacheNeeds
from ..parts import BuildContext, LayerCache, build_part, expected_tensors


class ModelParts:
    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        for e in spec.schedule:
            if not (0 <= e.layer < len(spec.layers) and 0 <= e.cache_of < len(spec.layers)):
                raise ValueError(f"schedule entry {e} names a layer outside 0..{len(spec.layers) - 1}")
        self.embedding = build_part("embedding", spec.embed, ctx)
        self.blocks = [build_part("block", layer, ctx) for layer in spec.layers]
        self.merges = {}                                   # a spec named by several runs is one part
        for e in spec.schedule:
            if e.before is not None and e.before not in self.merges:
                self.merges[e.before] = build_part("merge", e.before, ctx)
        self.tap = None                                    # a function (run, residual) called after every layer run, for inspection
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)

    def expected_tensors(self) -> Dict[str, tuple]:
        return expected_tensors(self.spec)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.load(tensors)
        for b in self.blocks:
            b.load(tensors)
        for m in self.merges.values():
            m.load(tensors)
        self.final_norm.load(tensors)
        self.head.load(tensors)

    def graph_safe(self) -> bool:
        """Whether every part only enqueues kernels, so that a decode step can be recorded."""
        return all(p.graph_safe for p in (self.embedding, self.final_norm, self.head, *self.blocks, *self.merges.values()))

    def cache_key(self, e) -> int:
        """The cache a run uses: the layer `cache_of` for the first replica, a number beyond the layers for the others."""
        return e.cache_of + e.replica * len(self.spec.layers)

    def cache_needs(self) -> Dict[int, CacheNeeds]:
        """What each cache keeps: one for every (layer named as `cache_of`, replica) of the schedule."""
        return {self.cache_key(e): self.blocks[e.cache_of].cache_needs() for e in self.spec.schedule}

    def forward(self, batch, cache_manager) -> torch.Tensor:
        """float32 logits [wanted rows, vocab] of a step."""
        if getattr(self.embedding, "needs_positions", False):
            x = self.embedding.forward(batch.ids, batch.positions)
        else:
            x = self.embedding.forward(batch.ids)
        schedule = self.spec.schedule
        x0 = None
        if self.merges:
            # the embedding's output is read again later, and the blocks update the stream in place
            x0, x = x, K.cast(x, torch.float32)
        h = None
        for i, e in enumerate(schedule):
            if e.before is not None:
                x, h = self.merges[e.before].forward(x, x0), None
            block = self.blocks[e.layer]
            ahead = i + 1 < len(schedule) and schedule[i + 1].before is None      # a rewritten stream is normed by its reader
            nxt = self.blocks[schedule[i + 1].layer].first_norm() if ahead else None
            cache = LayerCache(cache_manager, self.cache_key(e), owns=(e.cache_of == e.layer))
            x, h = block.forward(x, h, batch, cache, nxt)
            if self.tap is not None:
                self.tap(i, x)
        rows = K.gather_rows(x, batch.want_rows)
        return self.head.forward(self.final_norm.forward(rows))
