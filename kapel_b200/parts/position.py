"""Position encodings. A mixer owns one and asks it for what its kernels take.

kind "rope": theta^(-2j/r) frequencies (each divided by the spec's `divisor`), pairing (j, j + r/2), all in one table of (cos, sin)
per row made once a step with angles in 64-bit (crates/kapel-ops/src/rope.rs:63-101;
kernels/src/lib.rs rope_table :1092). kind "none": no rotation. With a `scaling` rule the frequencies
are made on the host in 64-bit (`scaled_frequencies`) and the table carries the rule's factor on cos
and sin. The pairing ("half" or "neighbours") is the consuming kernel's business: the table is one
(cos, sin) a pair either way.
"""
from __future__ import annotations

import math

import torch

from .. import kernels as K
from .base import Part


def scaled_frequencies(rotary_dim: int, theta: float, scaling):
    """(frequency of every pair as a list of floats, the factor on cos and sin) for `spec.RopeScaling`."""
    half = rotary_dim // 2
    f = [theta ** (-2.0 * j / rotary_dim) for j in range(half)]
    if scaling is None:
        return f, 1.0

    def pair_of(turns: float) -> float:
        return rotary_dim * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(scaling.fast)), 0)
    hi = min(math.ceil(pair_of(scaling.slow)), rotary_dim - 1)
    out = []
    for j in range(half):
        ramp = min(max((j - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[j] / scaling.factor * ramp + f[j] * (1.0 - ramp))
    return out, 0.1 * math.log(scaling.factor) + 1.0


class Rope(Part):
    graph_safe = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.pairing not in ("half", "neighbours"):
            raise ValueError(f"rope pairing {spec.pairing!r} is not built (\"half\", \"neighbours\")")
        scaling = getattr(spec, "scaling", None)
        if scaling is not None and not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0 and spec.theta > 1):
            raise ValueError(f"rope scaling {scaling} needs positive numbers and a base above 1")
        self._freqs = None
        if scaling is not None:                             # made when the part is built: a recorded step reads the same device tensor again
            f, magnitude = scaled_frequencies(spec.rotary_dim, float(spec.theta), scaling)
            divisor = float(getattr(spec, "divisor", 1.0))
            self._freqs = (torch.tensor([x / divisor for x in f], dtype=torch.float64).to(ctx.device), magnitude)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rope rotary_dim {spec.rotary_dim} must be positive and even")
        if not getattr(spec, "divisor", 1.0) > 0:
            raise ValueError(f"rope divisor {spec.divisor} must be positive")

    @property
    def rotary_dim(self) -> int:
        return self.spec.rotary_dim

    def tables(self, batch):
        """(cos, sin) [rows, rotary/2, 2] for this step's positions; shared by every layer with
        the same theta and rotary width."""
        divisor = float(getattr(self.spec, "divisor", 1.0))
        scaling = getattr(self.spec, "scaling", None)
        key = ("rope", float(self.spec.theta), int(self.spec.rotary_dim), divisor, scaling)
        if key not in batch.memo:
            if scaling is not None:
                batch.memo[key] = K.rope_table_freqs(batch.positions, self._freqs[0], self._freqs[1])
            else:
                batch.memo[key] = K.rope_table(batch.positions, self.spec.rotary_dim, self.spec.theta, divisor)
        return batch.memo[key]

    @property
    def neighbours(self) -> bool:
        return self.spec.pairing == "neighbours"


class NoPosition(Part):
    graph_safe = True

    rotary_dim = 0

    def tables(self, batch):
        return None
