"""Parts of category "merge": they rewrite the residual stream between two layer runs.

"input_mix": x <- W [x; x0], the stream and the embedding's output side by side through one
matrix [hidden, 2 hidden]; the result is a new float32 stream (the product's 32-bit sums are not
rounded on the way).

"input_add": x <- x + x0, in place on the float32 stream.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, linear, matrix_named


class InputMix(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        return {spec.weight: (spec.hidden, 2 * spec.hidden)}

    def load(self, tensors):
        self.weight = matrix_named(self.ctx, tensors, self.spec.weight)

    def forward(self, x, x0):
        """x, x0: float32 [rows, hidden]; returns the new stream, float32 [rows, hidden]."""
        both = K.concat2(x, x0, self.weight.dtype if self.weight.dtype == torch.float32 else self.ctx.dtype)
        return linear(self.ctx, both, self.weight, out_dtype=torch.float32)


class InputAdd(Part):
    graph_safe = True

    def forward(self, x, x0):
        """x, x0: float32 [rows, hidden]; x is updated in place and returned."""
        K.add_rmsnorm(x, x0, None, None, self.ctx.dtype)
        return x
