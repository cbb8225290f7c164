"""Attention with two score maps per head over the same values (kind "diff_attention").

Queries and keys hold two maps of ``head_dim`` columns per head, [map 1 | map 2]; every map is a causal softmax
attention of its own (rotary positions, a sliding window), and a head's output is

    o = a1 - lambda * a2,   o / sqrt(mean(o^2) + eps) * (1 - diff),   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff.

The cache keeps a key head per (key/value head, map), 2 G heads of ``head_dim`` columns, and G value heads: the two
maps of a key/value head read the same value rows (``KVRequest.v_heads``).  The query matrix's rows are put in the
order (key/value head, map, head of the group) when the weights are loaded, so that the 2 H maps are 2 H query heads
of an ordinary grouped-query attention over 2 G key heads and the library's attention kernels serve them as they
stand; a small kernel then joins each head's two results, norms and scales.  lambda is one number per layer and is
taken once, in 32-bit, when the weights are loaded.  With ``gate`` the product that makes q, k and v also makes
W_g h, and the joining kernel multiplies its result by sigmoid(W_g h), element by element.
"""

from __future__ import annotations

import math

import torch

from ..cache.cache import KVRequest
from .registry import build_part, register_part


class DiffAttention:
    @staticmethod
    def weight_shapes(spec):
        H, G, D, V, h = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_dim, spec.hidden_size
        shapes = {"q": (H * 2 * D, h), "k": (G * 2 * D, h), "v": (G * V, h), "o": (h, H * V)}
        shapes.update({n: (D,) for n in ("lq1", "lk1", "lq2", "lk2")})
        if getattr(spec, "gate", False):
            shapes["g"] = (H * V, h)
        return shapes

    def __init__(self, spec, weights, runtime):
        H, G, D = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if H % G:
            raise ValueError(f"{H} query heads cannot share {G} key/value heads evenly")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"window must be a positive number of positions, got {spec.window}")
        self.spec = spec
        self.ops = runtime.ops
        per = H // G
        # rows of W_q from (head, map) to (key/value head, map, head of the group)
        wq = weights["q"].reshape(G, per, 2, D, -1).permute(0, 2, 1, 3, 4).reshape(H * 2 * D, -1)
        self.gate = bool(getattr(spec, "gate", False))
        self.w_qkv = self.ops.prepare_matrix(torch.cat([wq, weights["k"], weights["v"]] + ([weights["g"]] if self.gate else []), dim=0))
        self.w_o = self.ops.prepare_matrix(weights["o"])
        f = {n: weights[n].float() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = (math.exp(float((f["lq1"] * f["lk1"]).sum())) - math.exp(float((f["lq2"] * f["lk2"]).sum()))
                    + float(spec.diff))
        self.position = build_part("position", spec.position, {}, runtime) if spec.position is not None else None
        self.scale = float(spec.scale)

    def cache_request(self):
        s = self.spec
        return KVRequest(num_kv_heads=2 * s.num_kv_heads, head_dim=s.head_dim, window=s.window, v_dim=s.v_dim,
                         v_heads=s.num_kv_heads)

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, layer_cache):
        s, ops = self.spec, self.ops
        H, G, D, V = s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim
        rows = h.shape[0]
        qkv = ops.linear(h, self.w_qkv)
        nq, nk = 2 * H * D, 2 * G * D
        q = qkv[:, :nq].view(rows, 2 * H, D)
        k = qkv[:, nq:nq + nk].view(rows, 2 * G, D)
        freqs, rot, mag = (None, 0, 1.0) if self.position is None else self.position.half_rotary()
        q = ops.rotate_half_store(ctx, q, k, qkv[:, nq + nk:nq + nk + G * V], layer_cache, freqs, rot, mag)
        a = ops.flex_attention(ctx, q, layer_cache, self.scale, v_dim=V, window=s.window)        # [rows, 2 H * V]
        if self.gate:
            o = ops.diff_combine(a, H, G, V, self.lam, float(s.norm_eps), 1.0 - float(s.diff), gate=qkv[:, nq + nk + G * V:])
        else:
            o = ops.diff_combine(a, H, G, V, self.lam, float(s.norm_eps), 1.0 - float(s.diff))
        return ops.linear(o, self.w_o)


register_part("mixer", "diff_attention", DiffAttention)
