"""A short causal convolution over time, added to its input (kind "causal_conv").

    out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)          (per channel; zeros before a sequence's start)

It reads the residual in the residual's own type and hands the run's dtype to the mixer behind it; the sum is 32-bit
and rounded once.  The last ``taps`` - 1 inputs of a sequence are its state: a 32-bit record per sequence and layer
in the cache's state group, zero when the sequence starts, so that a step of many tokens and the same tokens one by
one read the same inputs.
"""

from __future__ import annotations

from ..cache.cache import StateRequest
from .registry import register_part


class CausalConv:
    @staticmethod
    def weight_shapes(spec):
        return {"weight": (spec.size, spec.taps)}

    def __init__(self, spec, weights, runtime):
        if spec.taps < 1:
            raise ValueError(f"a convolution has at least one tap, got {spec.taps}")
        self.size, self.taps = int(spec.size), int(spec.taps)
        self.ops = runtime.ops
        self.dtype = runtime.dtype
        self.weight = weights["weight"].float().contiguous()     # 32-bit: it multiplies the 32-bit residual

    def cache_request(self):
        """The inputs that the next step's first rows look back to; a single tap looks back to nothing."""
        return StateRequest((self.taps - 1, self.size)) if self.taps > 1 else None

    def forward(self, ctx, x, layer_cache):
        state = layer_cache.state if layer_cache is not None else None
        return self.ops.causal_conv(ctx, x, self.weight, state, self.dtype)


register_part("conv", "causal_conv", CausalConv)
