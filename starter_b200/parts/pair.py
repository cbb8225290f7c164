"""Two mixers side by side (kind "pair"): both read the same normed rows, and the layer's mixer output is

    left_scale * left(h) + right_scale * right(h).

Each side is a mixer of its own kind with its own tensors and its own share of the layer's cache entry: the layer asks
the cache for everything both sides need (at most one of them keeps keys and values; the rest are state records), and
each side sees its part of the answer.  A side's scale multiplies what its output projection reads (32-bit, inside the
kernel that writes those rows).

Sides that can work from given projections (``heads_from``, with their matrices in ``joint``) share their products:
one product makes both sides' projections of the input, one small one the 32-bit pre-activations of both sides' gates,
both sides write their heads' outputs side by side into one buffer, and one product with [W_o left | W_o right] makes
the sum of the two output projections (the left side's bias, times its scale, joins it there).  Other sides run as they
are and their outputs are added.
"""

from __future__ import annotations

import torch

from ..cache.cache import KVRequest
from .registry import part_class, register_part


def _as_tuple(request):
    if request is None:
        return ()
    return request if isinstance(request, tuple) else (request,)


class PairMixer:
    @staticmethod
    def weight_shapes(spec):
        shapes = {}
        for side, sub in (("left", spec.left), ("right", spec.right)):
            for role, shape in part_class("mixer", sub.kind).weight_shapes(sub).items():
                shapes[f"{side}.{role}"] = shape
        return shapes

    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.ops = runtime.ops
        sides = []
        for side, sub, scale in (("left", spec.left, spec.left_scale), ("right", spec.right, spec.right_scale)):
            own = {role[len(side) + 1:]: w for role, w in weights.items() if role.startswith(side + ".")}
            cls = part_class("mixer", sub.kind)
            shares = hasattr(cls, "heads_from")
            sides.append(cls(sub, own, runtime, out_scale=float(scale), **({"own_products": False} if shares else {})))
        self.left, self.right = sides
        self.shared = all(getattr(side, "joint", None) is not None for side in sides)
        if self.shared:
            (l_in, l_gates, l_o), (r_in, r_gates, r_o) = self.left.joint, self.right.joint
            self.in_at = (0, l_in.shape[0], l_in.shape[0] + r_in.shape[0])
            self.w_in = self.ops.prepare_matrix(torch.cat([l_in, r_in], dim=0))
            gates = [g for g in (l_gates, r_gates) if g is not None]
            self.w_gates = self.ops.prepare_matrix(torch.cat(gates, dim=0)) if gates else None
            self.gate_at = (0, l_gates.shape[0] if l_gates is not None else 0)
            self.has_gates = (l_gates is not None, r_gates is not None)
            self.out_at = (0, l_o.shape[1], l_o.shape[1] + r_o.shape[1])
            self.w_o = self.ops.prepare_matrix(torch.cat([l_o, r_o], dim=1))
            self.o_bias = getattr(self.left, "o_bias", None)
            if getattr(self.right, "o_bias", None) is not None:
                self.o_bias = self.right.o_bias if self.o_bias is None else (self.o_bias + self.right.o_bias).contiguous()
            self.left.joint = self.right.joint = None
        else:
            for side in sides:
                if getattr(side, "joint", None) is not None:
                    raise ValueError("a mixer that hands its matrices to a pair needs a neighbour that does so too")
        left, right = _as_tuple(self.left.cache_request()), _as_tuple(self.right.cache_request())
        if any(isinstance(r, KVRequest) for r in right) or any(isinstance(r, KVRequest) for r in left[1:]):
            raise ValueError("of two mixers side by side only the left one may keep keys and values, as its first request")
        self._requests = left + right
        self._right_at = len(left)

    def children(self):
        """The two sides, for whoever walks a model's parts."""
        return (self.left, self.right)

    def cache_request(self):
        if not self._requests:
            return None
        return self._requests if len(self._requests) > 1 else self._requests[0]

    def prepare(self, cache) -> None:
        self.left.prepare(cache)
        self.right.prepare(cache)

    def forward(self, ctx, h, layer_cache):
        right_cache = layer_cache
        for _ in range(self._right_at):
            right_cache = right_cache.aux
        ops = self.ops
        if not self.shared:   # each side's output already carries its scale (and a side's bias its share of it)
            return ops.scaled_sum(self.left.forward(ctx, h, layer_cache), 1.0, self.right.forward(ctx, h, right_cache), 1.0)
        p = ops.linear(h, self.w_in)
        z = ops.linear(h, self.w_gates, out_float32=True) if self.w_gates is not None else None
        heads = torch.empty((h.shape[0], self.out_at[2]), dtype=h.dtype, device=h.device)
        self.left.heads_from(ctx, p[:, self.in_at[0]:self.in_at[1]], z if self.has_gates[0] else None, self.gate_at[0], layer_cache,
                             out=heads[:, self.out_at[0]:self.out_at[1]])
        self.right.heads_from(ctx, p[:, self.in_at[1]:self.in_at[2]], z if self.has_gates[1] else None, self.gate_at[1], right_cache,
                              out=heads[:, self.out_at[1]:self.out_at[2]])
        if self.o_bias is not None:
            return ops.linear_bias(heads, self.w_o, self.o_bias)
        return ops.linear(heads, self.w_o)


register_part("mixer", "pair", PairMixer)
