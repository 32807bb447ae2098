"""A mixture of small feed-forwards behind a router.

The router's product, scores, groups and choice are one kernel in 32-bit (the router's weight is
kept in float32 whatever the file holds); a second kernel lists the (token, k) pairs by expert;
the experts' two products run as grouped products over those lists (the activation is the first
one's epilogue), each pair's result in a row of its own; the last kernel adds a token's rows up in
the order of its choices with the router's weights. Nothing is read back to the host, so a step
with this feed-forward can be recorded. All experts' weights of a role are one tensor
[experts, out, in], each copied from the file straight into its rows. Gated experts
(down(act(gate h) * up h)) keep gate and up of an expert one below the other: the first grouped
product gives gate|up a pair, the gated unit's kernel the second product's input. A shared expert (a
feed-forward part of its own that every token runs) is added in the kernel that sums the experts up.
The gated activation "clamped_swish" bounds both halves: min(gate, L) sigmoid(a min(gate, L)) (clamp(up, -L, L) + 1).
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, require_product_widths, stack_rows
from .registry import build_part, part_class


class MoE(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.weights
        out = {w["router"]: (spec.experts, spec.hidden)}
        if w.get("correction"):
            out[w["correction"]] = (spec.experts,)
        for e in range(spec.experts):
            if spec.gated:
                out[w["gate"].format(e=e)] = (spec.intermediate, spec.hidden)
            out[w["up"].format(e=e)] = (spec.intermediate, spec.hidden)
            out[w["down"].format(e=e)] = (spec.hidden, spec.intermediate)
        if spec.shared is not None:
            out.update(part_class("feed_forward", spec.shared.kind).expected_tensors(spec.shared))
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.clamped = spec.gated and spec.activation == "clamped_swish"
        if self.clamped and not (spec.limit is not None and spec.limit > 0):
            raise ValueError(f"moe: the bounded gated unit needs a positive `limit`, got {spec.limit}")
        if not self.clamped and spec.activation not in (K.ACT_CODES if spec.gated else K.MOE_ACT_CODES):
            raise ValueError(f"moe: activation {spec.activation!r} is not built" + (" for gated experts" if spec.gated else ""))
        if spec.scoring not in K.ROUTE_SCORING:
            raise ValueError(f"moe: scoring {spec.scoring!r} is not built")
        self.shared = build_part("feed_forward", spec.shared, ctx) if spec.shared is not None else None
        if spec.experts % spec.groups or not 1 <= spec.keep_groups <= spec.groups:
            raise ValueError(f"moe: {spec.experts} experts in {spec.groups} groups of which {spec.keep_groups} are kept")
        if spec.keep_groups * (spec.experts // spec.groups) < spec.top or spec.top < 1:
            raise ValueError(f"moe: {spec.keep_groups} groups of {spec.experts // spec.groups} experts cannot give {spec.top}")

    def load(self, tensors):
        s, w = self.spec, self.spec.weights
        dev = self.ctx.device
        self.router = tensors[w["router"]].to(dev).float().contiguous()
        self.correction = tensors[w["correction"]].to(dev).float().contiguous() if w.get("correction") else None
        if s.gated:                    # an expert's gate rows, then its up rows
            names = [w[role].format(e=e) for e in range(s.experts) for role in ("gate", "up")]
            self.w_up = stack_rows(self.ctx, tensors, names, "moe").view(s.experts, 2 * s.intermediate, s.hidden)
        else:
            self.w_up = stack_rows(self.ctx, tensors, [w["up"].format(e=e) for e in range(s.experts)], "moe").view(
                s.experts, s.intermediate, s.hidden)
        if self.shared is not None:
            self.shared.load(tensors)
        self.w_down = stack_rows(self.ctx, tensors, [w["down"].format(e=e) for e in range(s.experts)], "moe").view(
            s.experts, s.hidden, s.intermediate)

    def forward(self, h):
        s = self.spec
        experts, weights = K.moe_route(h, self.router, self.correction, s.top, s.groups, s.keep_groups, s.group_top, s.scoring,
                                       s.renormalize)
        lists = K.moe_sort(experts, s.experts, self.w_up.dtype)
        if h.dtype != self.w_up.dtype:
            h = K.cast(h, self.w_up.dtype)
        also = self.shared.forward(h) if self.shared is not None else None
        if s.gated:
            both = K.moe_grouped(h, self.w_up, lists, "none", True, False, torch.float32)
            if self.clamped:
                inner = K.glu_clamped(both, s.limit, s.swish_alpha, out_dtype=self.w_up.dtype)
            else:
                inner = K.glu(both, s.activation, out_dtype=self.w_up.dtype)
        else:
            inner = K.moe_grouped(h, self.w_up, lists, s.activation, True, False, self.w_up.dtype)
        y = K.moe_grouped(inner, self.w_down, lists, "none", False, True, torch.float32)
        return K.moe_combine(y, weights, torch.float32, also=also)
