"""Two mixers side by side (kind "pair"): both read the same normed rows, and the layer's mixer output is

    left_scale * left(h) + right_scale * right(h).

Each side is a mixer of its own kind with its own tensors and its own share of the layer's cache entry: the layer asks
the cache for everything both sides need (at most one of them keeps keys and values; the rest are state records), and
each side sees its part of the answer.  A side's scale multiplies what its output projection reads (32-bit, inside the
kernel that writes those rows), so the two projections add up without a pass of their own over the scaled outputs.
"""

from __future__ import annotations

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
            sides.append(part_class("mixer", sub.kind)(sub, own, runtime, out_scale=float(scale)))
        self.left, self.right = sides
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
        # each side's output already carries its scale (and the left one's bias its share of it)
        return self.ops.scaled_sum(self.left.forward(ctx, h, layer_cache), 1.0, self.right.forward(ctx, h, right_cache), 1.0)


register_part("mixer", "pair", PairMixer)
