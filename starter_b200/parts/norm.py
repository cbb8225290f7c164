"""Root-mean-square norm (kind "rmsnorm").

Formula of the reference's kernels (engine/kernels/rmsnorm.py:31-45,
engine/kernels/add_rmsnorm.py:21-29): the mean of squares and the scaling are
32-bit; in bfloat16 the normalised value is rounded before the weight multiply.
"""

from __future__ import annotations

from .registry import register_part


class RMSNorm:
    @staticmethod
    def weight_shapes(spec):
        return {"weight": (spec.size,)}

    def __init__(self, spec, weights, runtime):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights["weight"]
        self.ops = runtime.ops

    def forward(self, x):
        return self.ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, x, delta):
        """x += delta in place (32-bit sum, stored in x's dtype), then the norm of the new x."""
        return self.ops.add_rmsnorm(x, delta, self.weight, self.eps)

    def folded(self, dtype):
        """(weight, eps) for a product that takes this norm in its prologue (``ops.linear(..., norm=)``), or None when
        the weight is kept in another type than the rows (a 32-bit weight in a bfloat16 run: the norm runs on its own)."""
        return (self.weight, self.eps) if self.weight.dtype == dtype else None


class GroupedRMSNorm:
    """Kind "grouped_rmsnorm": the row is cut into ``groups`` equal consecutive parts and each is divided by its own
    root mean square; all of it 32-bit, rounded once when the result is stored.  It reads rows of the residual's type
    (32-bit when the model keeps its residual so) and hands out rows of the run's dtype."""

    @staticmethod
    def weight_shapes(spec):
        return {"weight": (spec.size,)}

    def __init__(self, spec, weights, runtime):
        if spec.groups < 1 or spec.size % spec.groups:
            raise ValueError(f"a norm over {spec.size} columns cannot have {spec.groups} equal groups")
        self.size = spec.size
        self.groups = int(spec.groups)
        self.eps = float(spec.eps)
        self.weight = weights["weight"]
        if getattr(spec, "offset", 0.0):   # a weight stored around zero: offset + w, in 32-bit, once
            self.weight = (float(spec.offset) + self.weight.float()).contiguous()
        self.ops = runtime.ops
        self.dtype = runtime.dtype

    def forward(self, x):
        return self.ops.grouped_rmsnorm(x, (), self.weight, self.groups, self.eps, self.dtype)

    def add_forward(self, x, *deltas):
        """x += sum of the deltas, in place and in 32-bit (the deltas are summed first), then the norm of the new x."""
        return self.ops.grouped_rmsnorm(x, tuple(deltas), self.weight, self.groups, self.eps, self.dtype)


class BranchRMSNorm:
    """Kind "branch_rmsnorm": the norm of a branch's output on its way into the residual,
    x += y / sqrt(mean(y^2) + eps) * (offset + w) * s, in place and in 32-bit.  offset + w and the layer scale s are
    multiplied once at load.  ``add_to`` can hand back the new x rounded to the run's dtype: what the next branch reads
    when it reads the residual itself."""

    @staticmethod
    def weight_shapes(spec):
        shapes = {"weight": (spec.size,)}
        if spec.layer_scale:
            shapes["scale"] = (spec.size,)
        return shapes

    def __init__(self, spec, weights, runtime):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = (float(spec.offset) + weights["weight"].float()).contiguous()
        self.scale = weights["scale"].float().contiguous() if spec.layer_scale else None
        self.ops = runtime.ops
        self.dtype = runtime.dtype

    def add_to(self, x, y, want_rounded: bool = False, then=None):
        """x += norm(y) (* scale); returns the new x in the run's dtype when ``want_rounded`` (x itself if it has that type).
        ``then``: the norm that the next branch takes of the residual (kind "grouped_rmsnorm", one group); its result
        for the new x is returned instead, from the same kernel."""
        if then is not None:
            if self.scale is None and getattr(then, "groups", 0) == 1 and then.weight.dtype == x.dtype:
                return self.ops.branch_norm_add(x, y, self.weight, None, self.eps, self.dtype, next_norm=(then.weight, then.eps))
            self.ops.branch_norm_add(x, y, self.weight, self.scale, self.eps, None)
            return then.forward(x)
        return self.ops.branch_norm_add(x, y, self.weight, self.scale, self.eps, self.dtype if want_rounded else None)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "branch_rmsnorm", BranchRMSNorm)
register_part("norm", "grouped_rmsnorm", GroupedRMSNorm)
