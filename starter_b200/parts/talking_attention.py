"""Causal grouped-query attention whose scores meet across heads before the softmax (kind "talking_attention").

    q, k, v = W_q h, W_k h, W_v h                         (one product)
    q <- q / rms(q) * w_q,  k <- k / rms(k) * w_k         (over a token's WHOLE projection, all heads side by side)
    s_g(i, j) = cap * tanh(q_g(i) . k_c(g)(j) * scale / cap)
    t_h(i, j) = sum_g T[h, g] s_g(i, j)                   (a learned [heads, heads] table)
    visible:    j <= i and (i - j < window or j < keep_first)
    weights:    exp(t_h) / (sum over visible j of exp(t_h) + exp(sink_h))
    out = W_o [sum_j weights_h(i, j) v_c(h)(j)]_h

Nothing is rotated: positions enter through the mask only.  Norms, scores, the cap, the table, the softmax and its
weights are 32-bit in every run.  Each option is off when its spec field is None / False / 0.  A windowed layer asks
the cache for the pages that hold the kept first tokens plus a ring of pages for the window.
"""

from __future__ import annotations

import torch

from ..cache.cache import KVRequest
from .registry import register_part


class TalkingAttention:
    @staticmethod
    def weight_shapes(spec):
        H, G, D, V, h = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_dim, spec.hidden_size
        shapes = {"q": (H * D, h), "k": (G * D, h), "v": (G * V, h), "o": (h, H * V)}
        if spec.qk_norm_eps is not None:
            shapes.update({"q_norm": (H * D,), "k_norm": (G * D,)})
        if spec.talk:
            shapes["talk"] = (H, H)
        if spec.sink:
            shapes["sink"] = (H,)
        return shapes

    def __init__(self, spec, weights, runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads evenly")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"window must be a positive number of positions, got {spec.window}")
        if spec.keep_first < 0 or (spec.keep_first and spec.window is None):
            raise ValueError("kept first tokens go with a window")
        self.spec = spec
        self.ops = runtime.ops
        self.w_qkv = self.ops.prepare_matrix(torch.cat([weights["q"], weights["k"], weights["v"]], dim=0))
        self.w_o = self.ops.prepare_matrix(weights["o"])
        self.q_norm = self.k_norm = None
        if spec.qk_norm_eps is not None:
            self.q_norm = weights["q_norm"].float().contiguous()
            self.k_norm = weights["k_norm"].float().contiguous()
        self.talk = weights["talk"].float().contiguous() if spec.talk else None
        self.sink = weights["sink"].float().contiguous() if spec.sink else None

    def cache_request(self):
        s = self.spec
        return KVRequest(num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, window=s.window, v_dim=s.v_dim,
                         keep_first=s.keep_first if s.window is not None else 0)

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, layer_cache):
        s, ops = self.spec, self.ops
        qkv = ops.linear(h, self.w_qkv)
        q = ops.qk_norm_store(ctx, qkv, layer_cache, s.num_heads, self.q_norm, self.k_norm,
                              0.0 if s.qk_norm_eps is None else float(s.qk_norm_eps))
        a = ops.talking_attention(ctx, q, layer_cache, s.num_heads, float(s.scale), softcap=s.softcap, talk=self.talk,
                                  sink=self.sink, window=s.window, keep_first=s.keep_first)
        return ops.linear(a, self.w_o)


register_part("mixer", "talking_attention", TalkingAttention)
