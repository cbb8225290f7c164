"""The matrix memory of an mLSTM layer (kind "mlstm"): a [head_dim, v_dim] state per head with a normaliser and a
running maximum that keeps the exponential gates in range.

    q = W_q h / sqrt(head_dim),  k = W_k h,  v = W_v h
    i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))      (one pair per head)
    m_t = max(f + m_(t-1), i)                                                             (m starts at 0)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,   n_t the same with k alone
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    y = W_o (o / rms_head(o) * norm * sigmoid(W_g h))

One product makes q, k, v and the output gate in the run's dtype; a second, small one leaves the gates'
pre-activations as 32-bit numbers.  Gates, maxima, exponentials, the state, the division, the unit norm and the output
gate are 32-bit in the recurrence kernel.  A sequence's state (S, n and m of every head) is one 32-bit record in the
cache's state group, zero when the sequence starts; a step of many tokens leaves the record that the same tokens leave
one by one.  ``out_scale`` multiplies what the output projection reads (a mixer that stands beside another one passes
its share there).
"""

from __future__ import annotations

import torch

from ..cache.cache import StateRequest
from .registry import register_part


class MatrixMemory:
    @staticmethod
    def weight_shapes(spec):
        h, kd, vd, H = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_heads * spec.v_dim, spec.num_heads
        return {"q": (kd, h), "k": (kd, h), "v": (vd, h), "g": (vd, h), "o": (h, vd), "norm": (vd,),
                "i": (H, h), "i_bias": (H,), "f": (H, h), "f_bias": (H,)}

    def __init__(self, spec, weights, runtime, out_scale: float = 1.0, own_products: bool = True):
        if not spec.gate_cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {spec.gate_cap}")
        self.spec = spec
        self.ops = runtime.ops
        self.out_scale = float(out_scale)
        self.kd, self.vd = spec.num_heads * spec.head_dim, spec.num_heads * spec.v_dim
        # ``own_products`` False: the pair this mixer stands in makes one product of both sides' rows (see ``joint``)
        self.joint = (torch.cat([weights[n] for n in ("q", "k", "v", "g")], dim=0), torch.cat([weights["i"], weights["f"]], dim=0),
                      weights["o"])
        self.w_in = self.w_gates = self.w_o = None
        if own_products:
            self.w_in, self.w_gates, self.w_o = (self.ops.prepare_matrix(w) for w in self.joint)
            self.joint = None
        self.o_bias = None
        self.i_bias = weights["i_bias"].float().contiguous()
        self.f_bias = weights["f_bias"].float().contiguous()
        self.norm = weights["norm"].float().contiguous()

    def cache_request(self):
        s = self.spec
        return StateRequest(shape=(s.num_heads * s.head_dim * s.v_dim + s.num_heads * s.head_dim + s.num_heads,), dtype="float32")

    def prepare(self, cache) -> None:
        pass

    def heads_from(self, ctx, p, z, z_col, layer_cache, out=None):
        """From the projections p [rows, q | k | v | g] (a view of wider rows will do) and the gates' 32-bit
        pre-activations z[:, z_col : z_col + 2 heads] (input gates, then forget gates): what the output projection reads,
        times ``out_scale``, [rows, heads * v_dim]; into ``out`` when given (a view of wider rows)."""
        s, kd, vd = self.spec, self.kd, self.vd
        return self.ops.mlstm_scan(ctx, p[:, :kd], p[:, kd:2 * kd], p[:, 2 * kd:2 * kd + vd], p[:, 2 * kd + vd:2 * kd + 2 * vd], z, z_col,
                                   z_col + s.num_heads, self.i_bias, self.f_bias, float(s.gate_cap), self.norm, float(s.norm_eps),
                                   float(s.head_dim) ** -0.5, layer_cache.state, s.num_heads, s.head_dim, s.v_dim,
                                   out_scale=self.out_scale, out=out)

    def heads_output(self, ctx, h, layer_cache):
        return self.heads_from(ctx, self.ops.linear(h, self.w_in), self.ops.linear(h, self.w_gates, out_float32=True), 0, layer_cache)

    def forward(self, ctx, h, layer_cache):
        return self.ops.linear(self.heads_output(ctx, h, layer_cache), self.w_o)


register_part("mixer", "mlstm", MatrixMemory)
