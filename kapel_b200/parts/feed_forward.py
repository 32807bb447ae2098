"""The gated feed-forward: down(act(gate(h)) * up(h)), gate and up as one stacked product
(crates/kapel-models/src/model.rs:1429-1456; the gated unit kernels/src/lib.rs glu_any :2489); and
the plain one, down(act(up(h))), whose activation is a kernel of its own between the two products."""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, linear, matrix_named, stack_rows


class GatedMLP(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.weights
        return {
            w["gate"]: (spec.intermediate, spec.hidden),
            w["up"]: (spec.intermediate, spec.hidden),
            w["down"]: (spec.hidden, spec.intermediate),
        }

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.activation not in K.ACT_CODES:
            raise ValueError(f"gated_mlp: activation {spec.activation!r} is not built")
        # widths that are no multiple of 8 go through the products that pad their rows (`linear`), unfused
        self.fusable = spec.hidden % 8 == 0 and spec.intermediate % 8 == 0

    def load(self, tensors):
        w = self.spec.weights
        self.w_gate_up = stack_rows(self.ctx, tensors, [w["gate"], w["up"]], "gated_mlp")
        self.w_down = matrix_named(self.ctx, tensors, w["down"])

    def forward(self, h):
        # many rows of bfloat16: the gated unit is the epilogue of the gate|up product
        inner = K.gemm_glu_fused(h, self.w_gate_up, self.spec.activation) if (self.fusable and h.dtype == self.w_gate_up.dtype) else None
        if inner is None:
            gu = linear(self.ctx, h, self.w_gate_up, keep_split=True)
            inner = K.glu(gu, self.spec.activation, out_dtype=self.ctx.dtype)
        return linear(self.ctx, inner, self.w_down, keep_split=True)


class MLP(Part):
    """down(act(up(h))) without a gate; the activation reads the first product's sums in 32-bit
    (split over K or not) and leaves the second product's input."""

    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.weights
        return {w["up"]: (spec.intermediate, spec.hidden), w["down"]: (spec.hidden, spec.intermediate)}

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.activation not in K.PLAIN_ACT_CODES:
            raise ValueError(f"mlp: activation {spec.activation!r} is not built")

    def load(self, tensors):
        w = self.spec.weights
        self.w_up = matrix_named(self.ctx, tensors, w["up"])
        self.w_down = matrix_named(self.ctx, tensors, w["down"])

    def forward(self, h):
        up = linear(self.ctx, h, self.w_up, out_dtype=torch.float32, keep_split=True)
        inner = K.act(up, self.spec.activation, self.ctx.dtype)
        return linear(self.ctx, inner, self.w_down, keep_split=True)
