"""A layer's arrangement (kind "prenorm"): x += mixer(norm(x)); x += ff(norm(x)).

Order of the reference's layer (OPTIMIZATION_GUIDE.md:60-69,
engine/model.py:289-298).  Each branch leaves its output on the residual
stream; the sum is taken by the next norm.

Where the kernels can (``ops.folds``: the few rows of a decode step), a branch
takes both ends itself, as the reference's decode path does
(engine/model.py:186-210): a part with ``takes_fold`` gets ``residual=`` (the
stream, to which its last product adds its result, leaving the statistics of
the new rows in ``stream.stats``) and, once such statistics exist, the residual
un-normed together with ``norm=`` (weight, eps, statistics: what its first
product folds into its prologue).  A norm offers ``folded(dtype)`` for that;
parts or norms without these run the plain order.
"""

from __future__ import annotations

from .registry import build_part, register_part


class PreNormBlock:
    @staticmethod
    def sub_parts(spec):
        """(name, category, spec) of the parts this block is made of."""
        return (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer),
                ("ff_norm", "norm", spec.ff_norm), ("ff", "ff", spec.ff))

    def __init__(self, spec, weights, runtime):
        self.folds = getattr(runtime.ops, "folds", None)
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        self.ff.prepare(cache)

    def _branch(self, ctx, stream, norm, part, *args) -> None:
        fold = None
        if (self.folds is not None and getattr(part, "takes_fold", False) and hasattr(norm, "folded")
                and self.folds(stream.x.shape[0], stream.x.dtype)):
            fold = norm.folded(stream.x.dtype)
        if fold is None:
            stream.push(part.forward(ctx, stream.normed(norm), *args))
        elif stream.pending is None and stream.stats is not None:
            part.forward(ctx, stream.x, *args, norm=fold + (stream.stats,), residual=stream)
        else:   # nothing has left the rows' statistics yet (a model's first branch): the norm runs on its own
            part.forward(ctx, stream.normed(norm), *args, residual=stream)

    def forward(self, ctx, stream, layer_cache) -> None:
        self._branch(ctx, stream, self.mixer_norm, self.mixer, layer_cache)
        self._branch(ctx, stream, self.ff_norm, self.ff)


class ParallelBlock:
    """Kind "parallel": one norm, read by the mixer and by the feed-forward; x += mixer(n) + ff(n).  Both outputs
    wait on the residual stream and are added, in the residual's own type, by the next norm.  ``ff`` may be absent."""

    @staticmethod
    def sub_parts(spec):
        parts = (("norm", "norm", spec.norm), ("mixer", "mixer", spec.mixer))
        return parts + ((("ff", "ff", spec.ff),) if spec.ff is not None else ())

    def __init__(self, spec, weights, runtime):
        self.ff = None
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        if self.ff is not None:
            self.ff.prepare(cache)

    def forward(self, ctx, stream, layer_cache) -> None:
        n = stream.normed(self.norm)
        outputs = [self.mixer.forward(ctx, n, layer_cache)]
        if self.ff is not None:
            outputs.append(self.ff.forward(ctx, n))
        stream.push(*outputs)


class PostNormBlock:
    """Kind "postnorm": the branches read the residual itself and are normed on the way back,
    x += N1(mixer(conv(x))); x += N2(ff(x)).  The residual is one 32-bit tensor, changed in place by the branch norms
    (kind "branch_rmsnorm"); the mixer reads it through the ``conv`` part (or rounded to the run's dtype when there is
    none), the feed-forward reads the rounded copy that the mixer's branch norm hands back.  The layer's cache entry
    holds the mixer's keys and values and, beside them (``aux``), the conv part's state."""

    @staticmethod
    def sub_parts(spec):
        parts = (("mixer", "mixer", spec.mixer), ("mixer_norm", "norm", spec.mixer_norm))
        if spec.conv is not None:
            parts += (("conv", "conv", spec.conv),)
        if spec.ff is not None:
            parts += (("ff", "ff", spec.ff), ("ff_norm", "norm", spec.ff_norm))
        return parts

    def __init__(self, spec, weights, runtime):
        self.conv = self.ff = self.ff_norm = None
        self.dtype = runtime.dtype
        self.ops = runtime.ops
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        main = self.mixer.cache_request()
        state = self.conv.cache_request() if self.conv is not None else None
        return main if state is None else (main, state)

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        if self.ff is not None:
            self.ff.prepare(cache)

    def forward(self, ctx, stream, layer_cache) -> None:
        x = stream.x
        if stream.pending is not None:
            raise RuntimeError("a layer of this kind adds its branches itself; nothing may wait on the residual")
        if self.conv is not None:
            h = self.conv.forward(ctx, x, getattr(layer_cache, "aux", None))
        else:
            h = x if x.dtype == self.dtype else self.ops.cast_rows(x, self.dtype)
        rounded = self.mixer_norm.add_to(x, self.mixer.forward(ctx, h, layer_cache), want_rounded=self.ff is not None)
        if self.ff is not None:
            self.ff_norm.add_to(x, self.ff.forward(ctx, rounded))


class SandwichBlock:
    """Kind "sandwich": every branch is normed on the way in and on the way back,
    x += N1b(mixer(N1(x))); x += N2b(ff(N2(x))).  The residual is one 32-bit tensor, changed in place by the outer norms
    (kind "branch_rmsnorm"); the inner norms (kind "grouped_rmsnorm") read it and hand the run's dtype to the branch.  The
    kernel that adds the mixer's normed output also norms the new residual for the feed-forward."""

    @staticmethod
    def sub_parts(spec):
        parts = (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer), ("mixer_out_norm", "norm", spec.mixer_out_norm))
        if spec.ff is not None:
            parts += (("ff_norm", "norm", spec.ff_norm), ("ff", "ff", spec.ff), ("ff_out_norm", "norm", spec.ff_out_norm))
        return parts

    def __init__(self, spec, weights, runtime):
        self.ff = self.ff_norm = self.ff_out_norm = None
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        if self.ff is not None:
            self.ff.prepare(cache)

    def forward(self, ctx, stream, layer_cache) -> None:
        x = stream.x
        if stream.pending is not None:
            raise RuntimeError("a layer of this kind adds its branches itself; nothing may wait on the residual")
        y = self.mixer.forward(ctx, self.mixer_norm.forward(x), layer_cache)
        if self.ff is None:
            self.mixer_out_norm.add_to(x, y)
            return
        h = self.mixer_out_norm.add_to(x, y, then=self.ff_norm)    # the mixer's way back and the feed-forward's way in: one kernel
        self.ff_out_norm.add_to(x, self.ff.forward(ctx, h))


register_part("block", "prenorm", PreNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
