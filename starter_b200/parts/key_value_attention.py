"""Causal grouped-query attention whose values are its keys (kind "key_value_attention").

    q, k = W_q h + b_q, W_k h + b_k                           (one product; the biases join in the next kernel)
    q, k <- short causal convolution over time, per channel   (y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start)
    v = k                                                     (as it leaves the convolution)
    q, k <- per head: x / rms(x) * weight                     (a weight of head_dim values, shared by the heads)
    q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))      (p the position)
    weights = exp(s_j) / (1 + sum_j exp(s_j)),  s = q . k * scale over the keys j <= p
    out = W_o [sigmoid(W_g h)_h * sum_j weights_h(j) v_c(h)(j)]_h + b_o

Nothing is rotated.  The cache keeps the normed keys in its key rows and the keys before the norm in its value rows;
the last ``taps`` - 1 biased projections of a sequence are a 32-bit record in the cache's state group, so that a step of
many tokens and the same tokens one by one read the same inputs.  Biases, the convolution, norms, the temperature,
scores, the softmax and the gate are 32-bit in every run; the gate's product leaves 32-bit numbers.  Every option is
off when its spec field is None / False / 0.  ``out_scale`` multiplies the heads' outputs before the projection (a
mixer that stands beside another one passes its share there); the bias then takes it as well.
"""

from __future__ import annotations

import torch

from ..cache.cache import KVRequest, StateRequest
from .registry import register_part


class KeyValueAttention:
    @staticmethod
    def weight_shapes(spec):
        H, G, D, h = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.hidden_size
        shapes = {"q": (H * D, h), "k": (G * D, h), "o": (h, H * D)}
        if spec.bias:
            shapes.update({"q_bias": (H * D,), "k_bias": (G * D,), "o_bias": (h,)})
        if spec.taps:
            shapes.update({"q_conv": (H * D, spec.taps), "k_conv": (G * D, spec.taps)})
        if spec.qk_norm_eps is not None:
            shapes.update({"q_norm": (D,), "k_norm": (D,)})
        if spec.head_gate:
            shapes["g"] = (H, h)
        return shapes

    def __init__(self, spec, weights, runtime, out_scale: float = 1.0, own_products: bool = True):
        H, G, D = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if H % G:
            raise ValueError(f"{H} query heads cannot share {G} key/value heads evenly")
        if spec.taps < 0 or spec.temp_every < 0:
            raise ValueError("taps and the temperature's step count from zero")
        self.spec = spec
        self.ops = runtime.ops
        self.out_scale = float(out_scale)
        dev = weights["q"].device

        def f32(name):
            return weights[name].float().contiguous()

        # ``own_products`` False: a mixer that stands beside another one hands its matrices to the pair, which makes one
        # product of both sides' rows (``joint``: rows of the input product, rows of the 32-bit gate product, W_o)
        self.joint = (torch.cat([weights["q"], weights["k"]], dim=0), weights["g"] if spec.head_gate else None, weights["o"])
        self.w_qk = self.w_o = self.w_g = None
        if own_products:
            self.w_qk = self.ops.prepare_matrix(self.joint[0])
            self.w_o = self.ops.prepare_matrix(weights["o"])
            self.w_g = self.ops.prepare_matrix(weights["g"]) if spec.head_gate else None
            self.joint = None
        self.q_bias = f32("q_bias") if spec.bias else None
        self.k_bias = f32("k_bias") if spec.bias else None
        self.o_bias = (f32("o_bias") * self.out_scale).contiguous() if spec.bias else None
        self.q_conv = f32("q_conv") if spec.taps else None
        self.k_conv = f32("k_conv") if spec.taps else None
        self.q_norm = self.k_norm = None
        self.eps = 0.0
        if spec.qk_norm_eps is not None:
            self.q_norm, self.k_norm, self.eps = f32("q_norm"), f32("k_norm"), float(spec.qk_norm_eps)
        self.sink = torch.zeros(H, dtype=torch.float32, device=dev) if spec.unit_sink else None

    def cache_request(self):
        s = self.spec
        kv = KVRequest(num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, v_dim=s.head_dim)
        if s.taps > 1:
            return (kv, StateRequest((s.taps - 1, (s.num_heads + s.num_kv_heads) * s.head_dim)))
        return kv

    def prepare(self, cache) -> None:
        pass

    def heads_from(self, ctx, qk, z, z_col, layer_cache, out=None):
        """From the projections qk [rows, (heads + kv heads) * head_dim] (a view of wider rows will do) and the gates'
        32-bit pre-activations z[:, z_col : z_col + heads]: the gated heads' outputs times ``out_scale``, [rows, heads *
        head_dim], before the output projection; into ``out`` when given (a view of wider rows)."""
        s, ops = self.spec, self.ops
        H, D = s.num_heads, s.head_dim
        state = layer_cache.aux.state if s.taps > 1 else None
        q = ops.conv_qk_store(ctx, qk[:, :H * D], qk[:, H * D:], layer_cache, state, H, self.q_bias, self.k_bias, self.q_conv,
                              self.k_conv, self.q_norm, self.k_norm, self.eps, float(s.temp_coef), int(s.temp_every))
        a = ops.flex_attention(ctx, q, layer_cache, float(s.scale), v_dim=D, sink=self.sink)
        if z is None:
            if self.out_scale == 1.0 and out is None:
                return a
            raise NotImplementedError("a share of the output without a head gate is not built")
        return ops.head_gate(a, z, z_col, H, self.out_scale, out=out)

    def heads_output(self, ctx, h, layer_cache):
        z = self.ops.linear(h, self.w_g, out_float32=True) if self.w_g is not None else None
        return self.heads_from(ctx, self.ops.linear(h, self.w_qk), z, 0, layer_cache)

    def forward(self, ctx, h, layer_cache):
        o = self.heads_output(ctx, h, layer_cache)
        if self.o_bias is not None:
            return self.ops.linear_bias(o, self.w_o, self.o_bias)
        return self.ops.linear(o, self.w_o)


register_part("mixer", "key_value_attention", KeyValueAttention)
