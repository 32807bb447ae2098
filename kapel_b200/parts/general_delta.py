"""The generalized delta rule as a mixer with a state of its own.

One stacked product gives r | k | v | g | a | w1 in 32-bit (w1: the hidden layer of the small net
behind the decay). The scan's kernels finish the decay (tanh, the net's second layer, sigmoid, the
exponential) and the removal rate per head and key channel, make the unit keys, and walk each
request's rows in order from the memory its slot holds, leaving the memory of the request's last row
there. Then each head's read-out is divided by its root mean square, times a weight over all heads,
times sigmoid(g), and the output product follows. Prompt portions and single tokens take the same
kernels: a step's rows of one request are a run of the recurrence, however the prompt was cut.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, StateSpec
from .base import Part, linear, matrix_named, pad_columns, product_width, stack_rows


class GeneralDelta(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w, n = spec.weights, spec.num_heads * spec.head_dim
        out = {w[r]: (n, spec.hidden) for r in ("r", "k", "v", "g", "a")}
        out.update({w["a_bias"]: (n,), w["w1"]: (spec.lora, spec.hidden), w["w2"]: (n, spec.lora), w["w0"]: (n,), w["norm"]: (n,),
                    w["o"]: (spec.hidden, n)})
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.head_dim > 256:
            raise ValueError(f"general_delta: a key size of {spec.head_dim} is more than the scan kernel's 256")
        if spec.lora < 1:
            raise ValueError(f"general_delta: a decay net of {spec.lora} hidden values")

    def load(self, tensors):
        w = self.spec.weights
        self.w_in = stack_rows(self.ctx, tensors, [w[r] for r in ("r", "k", "v", "g", "a", "w1")], "general_delta")
        self.w_o = pad_columns(self.ctx, matrix_named(self.ctx, tensors, w["o"]))      # the gate kernel writes rows this wide
        dev = self.ctx.device
        f32 = lambda n: tensors[n].to(dev).float().contiguous()
        self.w2, self.w0, self.a_bias = f32(w["w2"]).t().contiguous(), f32(w["w0"]), f32(w["a_bias"])      # the second layer turned: [lora, heads d]
        n = tensors[w["norm"]].to(dev)
        self.norm_weight = n.float().contiguous() if self.ctx.is_f32 else n.contiguous()

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(state=StateSpec((s.num_heads * s.head_dim * s.head_dim,)))

    def forward(self, h, batch, cache):
        s = self.spec
        n = s.num_heads * s.head_dim
        stacked = linear(self.ctx, h, self.w_in, out_dtype=torch.float32, keep_split=True)
        o = K.gdelta_scan(stacked, 0, n, 2 * n, 4 * n, 5 * n, self.w2, self.w0, self.a_bias, s.decay_scale, s.unit_eps, cache.state(),
                          batch.entry_ranges(), batch.slots, batch.entries, s.num_heads, s.head_dim)
        y = K.head_gate(o, stacked, 3 * n, self.norm_weight, True, s.eps, self.ctx.dtype, pad_to=product_width(self.ctx, n))
        return linear(self.ctx, y, self.w_o, keep_split=True)
