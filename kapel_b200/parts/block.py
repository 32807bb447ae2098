"""How a layer's parts are arranged.

"sandwich" (Gemma 2; crates/kapel-models/src/model.rs:1401-1460):
    h = pre_mixer(x); a = mixer(h); x += post_mixer(a); h = pre_ffn(x); m = ffn(h); x += post_ffn(m)
    (a layer without a feed-forward ends after the first sum)
"prenorm": the same without the post norms.
"postnorm": the branches read the residual itself (rounded to the activation dtype), and only their
    outputs are normed: x += post_mixer(mixer(x)); x += post_ffn(ffn(x)); a layer may have no
    feed-forward.

"parallel": one norm, and both branches read its output h: x += s1 * mixer(shift(h)) + s2 * ffn(h), with
    an optional weight a channel on each branch and an optional token shift ahead of the mixer (the row
    before a request's first row of a step is kept in the layer's state).

The residual x is float32 and is updated in place. Each sum is one kernel together with the
norm before it and the norm after it, when those are RMS norms.
"""
from __future__ import annotations

from .. import kernels as K
from .base import Part
from .norm import add_branch
from .registry import build_part


class SandwichBlock(Part):
    norm_roles = ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")

    @classmethod
    def roles_of(cls, spec):
        """The norms a layer of this arrangement has: without a feed-forward, those around the mixer."""
        return cls.norm_roles if spec.ffn is not None else tuple(r for r in cls.norm_roles if r.endswith("_mixer"))

    @classmethod
    def expected_tensors(cls, spec):
        from .registry import part_class

        out = {}
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        if spec.ffn is not None:
            out.update(part_class("feed_forward", spec.ffn.kind).expected_tensors(spec.ffn))
        for role in cls.roles_of(spec):
            n = spec.norms[role]
            out.update(part_class("norm", n.kind).expected_tensors(n))
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        roles = self.roles_of(spec)
        missing = [r for r in roles if r not in spec.norms]
        if missing:
            raise ValueError(f"{spec.kind} block: norms {missing} are missing")
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ffn = build_part("feed_forward", spec.ffn, ctx) if spec.ffn is not None else None
        self.norms = {r: build_part("norm", spec.norms[r], ctx) for r in roles}

    @property
    def graph_safe(self) -> bool:
        parts = [self.mixer, *self.norms.values()] + ([self.ffn] if self.ffn is not None else [])
        return all(p.graph_safe for p in parts)

    def cache_needs(self):
        """What this layer keeps between steps: its mixer's pages and state."""
        return self.mixer.cache_needs()

    def first_norm(self):
        """The norm this block applies to the residual first; the block before it may apply it on
        the way and hand the result in as `h`."""
        return self.norms["pre_mixer"]

    def load(self, tensors):
        self.mixer.load(tensors)
        if self.ffn is not None:
            self.ffn.load(tensors)
        for n in self.norms.values():
            n.load(tensors)

    def forward(self, x, h, batch, cache, next_norm):
        if h is None:
            h = self.norms["pre_mixer"].forward(x)
        a = self.mixer.forward(h, batch, cache)
        if self.ffn is None:
            return x, add_branch(self.ctx, x, a, self.norms.get("post_mixer"), next_norm)
        h = add_branch(self.ctx, x, a, self.norms.get("post_mixer"), self.norms["pre_ffn"])
        m = self.ffn.forward(h)
        h_next = add_branch(self.ctx, x, m, self.norms.get("post_ffn"), next_norm)
        return x, h_next


class PreNormBlock(SandwichBlock):
    norm_roles = ("pre_mixer", "pre_ffn")


class PostNormBlock(Part):
    """Each branch reads the residual and is normed on its way back into it."""

    @classmethod
    def expected_tensors(cls, spec):
        from .registry import part_class

        out = {}
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        if spec.ffn is not None:
            out.update(part_class("feed_forward", spec.ffn.kind).expected_tensors(spec.ffn))
        for role in cls.roles_of(spec):
            n = spec.norms[role]
            out.update(part_class("norm", n.kind).expected_tensors(n))
        return out

    @staticmethod
    def roles_of(spec):
        return ("post_mixer", "post_ffn") if spec.ffn is not None else ("post_mixer",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        missing = [r for r in self.roles_of(spec) if r not in spec.norms]
        if missing:
            raise ValueError(f"{spec.kind} block: norms {missing} are missing")
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ffn = build_part("feed_forward", spec.ffn, ctx) if spec.ffn is not None else None
        self.norms = {r: build_part("norm", spec.norms[r], ctx) for r in self.roles_of(spec)}

    @property
    def graph_safe(self) -> bool:
        parts = [self.mixer, *self.norms.values()] + ([self.ffn] if self.ffn is not None else [])
        return all(p.graph_safe for p in parts)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def first_norm(self):
        return None                     # the mixer reads the residual as it is

    def load(self, tensors):
        self.mixer.load(tensors)
        if self.ffn is not None:
            self.ffn.load(tensors)
        for n in self.norms.values():
            n.load(tensors)

    def _read(self, x):
        return x if self.ctx.is_f32 else K.cast(x, self.ctx.dtype)

    def forward(self, x, h, batch, cache, next_norm):
        """`h`, where given, is the residual already in the activation dtype: the block before left it
        with its last sum (this block's `first_norm()` is None, so the engine never norms ahead)."""
        narrow = not self.ctx.is_f32                         # the branches read a rounded copy of the residual
        a = self.mixer.forward(h if (h is not None and narrow) else self._read(x), batch, cache)
        last = self.ffn is None
        h = add_branch(self.ctx, x, a, self.norms["post_mixer"], next_norm if last else None, copy_out=narrow)
        if last:
            return x, h
        m = self.ffn.forward(h if narrow else x)
        return x, add_branch(self.ctx, x, m, self.norms["post_ffn"], next_norm, copy_out=narrow)


class ParallelBlock(Part):
    """x <- x + (s1 * mixer(shift(h)) + s2 * ffn(h)) with h = pre(x): one norm, two branches that read it.
    The branches' weighted sum is one kernel (32-bit), the residual sum and the next layer's norm another."""

    @classmethod
    def expected_tensors(cls, spec):
        from .registry import part_class

        out = {}
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        if spec.ffn is not None:
            out.update(part_class("feed_forward", spec.ffn.kind).expected_tensors(spec.ffn))
        n = spec.norms["pre"]
        out.update(part_class("norm", n.kind).expected_tensors(n))
        for name in (spec.scales or ()):
            if name is not None:
                out[name] = (n.width,)
        if spec.shift is not None:
            out[spec.shift] = (n.width,)
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if "pre" not in spec.norms:
            raise ValueError("parallel block: the norm `pre` is missing")
        self.width = spec.norms["pre"].width
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ffn = build_part("feed_forward", spec.ffn, ctx) if spec.ffn is not None else None
        self.norm = build_part("norm", spec.norms["pre"], ctx)
        if spec.scales is not None and (len(spec.scales) != 2 or spec.scales[0] is None or (spec.scales[1] is None) != (spec.ffn is None)):
            raise ValueError(f"parallel block: branch weights {spec.scales} for a layer with{'out' if spec.ffn is None else ''} a feed-forward")

    @property
    def graph_safe(self) -> bool:
        parts = [self.mixer, self.norm] + ([self.ffn] if self.ffn is not None else [])
        return all(p.graph_safe for p in parts)

    def cache_needs(self):
        from ..cache import CacheNeeds, StateSpec

        needs = self.mixer.cache_needs().named("mixer")
        if self.spec.shift is not None:
            needs = needs.merged(CacheNeeds(states=(("shift", StateSpec((self.width,))),)))
        return needs

    def first_norm(self):
        return self.norm

    def load(self, tensors):
        import torch

        self.mixer.load(tensors)
        if self.ffn is not None:
            self.ffn.load(tensors)
        self.norm.load(tensors)
        dev = self.ctx.device
        f32 = lambda name: tensors[name].to(dev).float().contiguous()
        one = lambda: torch.ones((self.width,), dtype=torch.float32, device=dev)
        names = self.spec.scales or (None, None)
        self.scale_mixer = f32(names[0]) if names[0] is not None else one()
        self.scale_ffn = (f32(names[1]) if names[1] is not None else one()) if self.ffn is not None else None
        self.shift = f32(self.spec.shift) if self.spec.shift is not None else None

    def forward(self, x, h, batch, cache, next_norm):
        if h is None:
            h = self.norm.forward(x)
        hm = h
        if self.shift is not None:
            hm = K.token_shift(h, self.shift, cache.state_of("shift"), batch.row_entry, batch.entry_ranges(), batch.slots, batch.entries,
                               keep=cache.owns)
        a = self.mixer.forward(hm, batch, cache.scoped("mixer"))
        m = self.ffn.forward(h) if self.ffn is not None else None
        both = K.weighted_sum2(a, self.scale_mixer, m, self.scale_ffn)
        return x, add_branch(self.ctx, x, both, None, next_norm)
