"""Gated linear attention with tied gates, the input gate being one minus the forget gate (HGRN2), as a mixer with a state
of its own.

One stacked product gives q | f | v in 32-bit. The scan's kernels apply silu to q, make the gate
f = l + (1 - l) sigmoid(f + bias) with its lower bound l per head and channel, and walk each request's
rows in order from the memory its slot holds: S <- diag(f) S + (1 - f) v^T, o = S^T q. Then each
head's read-out is RMS-normed over its value size with one weight for all heads, and the output
product follows. Prompt portions and single tokens take the same kernels.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, StateSpec
from .base import Part, linear, matrix_named, pad_columns, product_width, stack_rows


class ForgetGate(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w, nq, nv = spec.weights, spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim
        return {w["q"]: (nq, spec.hidden), w["f"]: (nq, spec.hidden), w["f_bias"]: (nq,), w["lower"]: (nq,), w["v"]: (nv, spec.hidden),
                w["norm"]: (spec.v_head_dim,), w["o"]: (spec.hidden, nv)}

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.head_dim > 256:
            raise ValueError(f"forget_gate: a key size of {spec.head_dim} is more than the scan kernel's 256")

    def load(self, tensors):
        s, w = self.spec, self.spec.weights
        self.w_in = stack_rows(self.ctx, tensors, [w["q"], w["f"], w["v"]], "forget_gate")
        self.w_o = pad_columns(self.ctx, matrix_named(self.ctx, tensors, w["o"]))
        dev = self.ctx.device
        f32 = lambda n: tensors[n].to(dev).float().contiguous()
        self.f_bias, self.lower = f32(w["f_bias"]), f32(w["lower"])
        n = tensors[w["norm"]].to(dev)
        n = n.float() if self.ctx.is_f32 else n
        self.norm_weight = n.repeat(s.num_heads).contiguous()                           # one weight for all heads

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(state=StateSpec((s.num_heads * s.head_dim * s.v_head_dim,)))

    def forward(self, h, batch, cache):
        s = self.spec
        nq, nv = s.num_heads * s.head_dim, s.num_heads * s.v_head_dim
        stacked = linear(self.ctx, h, self.w_in, out_dtype=torch.float32, keep_split=True)
        o = K.gate_scan(stacked, 0, nq, 2 * nq, self.f_bias, self.lower, cache.state(), batch.entry_ranges(), batch.slots, batch.entries,
                        s.num_heads, s.head_dim, s.v_head_dim)
        y = K.head_gate(o, stacked, 0, self.norm_weight, True, s.eps, self.ctx.dtype, pad_to=product_width(self.ctx, nv), gate_act="none")
        return linear(self.ctx, y, self.w_o, keep_split=True)
