"""Two mixers side by side that read the same input: left_scale * left(h) + right_scale * right(h).

Each side keeps what it keeps under its own name in the layer's cache (`CacheNeeds.named`), and sees
the cache through that name (`LayerCache.scoped`); at most one side asks for pages. The weighted sum
is one kernel in 32-bit; a side whose output product has a bias that it can leave to its caller
(`forward_unbiased` and `out_bias`) has it added there.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part
from .registry import build_part, part_class


class ParallelMixer(Part):
    @staticmethod
    def expected_tensors(spec):
        out = {}
        for side in (spec.left, spec.right):
            out.update(part_class("mixer", side.kind).expected_tensors(side))
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.left = build_part("mixer", spec.left, ctx)
        self.right = build_part("mixer", spec.right, ctx)
        self.cache_needs()                      # refuses two sides that both want pages

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)
        s, dev = self.spec, self.ctx.device
        width = s.left.hidden
        self.va = torch.full((width,), float(s.left_scale), dtype=torch.float32, device=dev)
        self.vb = torch.full((width,), float(s.right_scale), dtype=torch.float32, device=dev)
        self.vc = None
        for side, scale in ((self.left, s.left_scale), (self.right, s.right_scale)):
            bias = getattr(side, "out_bias", None) if hasattr(side, "forward_unbiased") else None
            if bias is not None:
                self.vc = bias.float() * float(scale) + (self.vc if self.vc is not None else 0.0)
        if self.vc is not None:
            self.vc = self.vc.contiguous()

    def cache_needs(self):
        return self.left.cache_needs().named("left").merged(self.right.cache_needs().named("right"))

    def forward(self, h, batch, cache):
        run = lambda side, name: (side.forward_unbiased if hasattr(side, "forward_unbiased") else side.forward)(h, batch, cache.scoped(name))
        return K.weighted_sum2(run(self.left, "left"), self.va, run(self.right, "right"), self.vb, self.vc)
