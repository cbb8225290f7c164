"""Dense gated feed-forward (kind "gated_mlp"): down(silu(gate(x)) * up(x)), or with the activation
"clamped_swish" down(g * sigmoid(alpha g) * (u + 1)) for g = min(gate(x), limit), u = clamp(up(x), -limit, limit).

The reference fuses gate and up into one [2I, H] matrix, gate half first
(engine/model.py:116, engine/kernels/swiglu.py:5-6), and rounds gate, up,
silu(gate) and the product to bfloat16 (engine/kernels/swiglu.py:21-24).
"""

from __future__ import annotations

import torch

from .registry import register_part


class GatedMLP:
    @staticmethod
    def weight_shapes(spec):
        return {
            "gate": (spec.intermediate_size, spec.hidden_size),
            "up": (spec.intermediate_size, spec.hidden_size),
            "down": (spec.hidden_size, spec.intermediate_size),
        }

    def __init__(self, spec, weights, runtime):
        if spec.activation not in ("silu", "clamped_swish"):
            raise ValueError(f"activation {spec.activation!r} is not built; 'silu' and 'clamped_swish' are")
        self.activation = spec.activation
        if self.activation == "clamped_swish":
            if spec.limit is None or not spec.limit > 0:
                raise ValueError("the clamped activation needs a positive limit")
            self.limit, self.alpha = float(spec.limit), float(spec.alpha)
        self.hidden_size = spec.hidden_size
        self.intermediate_size = spec.intermediate_size
        self.ops = runtime.ops
        self.w_gate_up = self.ops.prepare_matrix(torch.cat([weights["gate"], weights["up"]], dim=0), halves=2)
        self.w_down = self.ops.prepare_matrix(weights["down"])
        self.takes_fold = self.activation == "silu" and spec.hidden_size % 8 == 0 and spec.intermediate_size % 8 == 0

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, norm=None, residual=None):
        """h is the normed input; with ``norm`` it is the residual itself and the norm is taken inside the first
        product; with ``residual`` the result is added to that tensor instead of being returned on its own."""
        if self.activation == "clamped_swish":
            return self.ops.linear(self.ops.linear_gated_clamp(h, self.w_gate_up, self.alpha, self.limit), self.w_down)
        if norm is None and residual is None:
            return self.ops.linear(self.ops.linear_swiglu(h, self.w_gate_up), self.w_down)
        act = self.ops.linear_swiglu(h, self.w_gate_up, norm=norm)
        return self.ops.linear(act, self.w_down, add_to=residual)


class ActMLP:
    """Kind "act_mlp": down(act(up(x))) without a gate.  "xielu": act(z) = a+ z^2 + z / 2 for z > 0 and
    a- (exp(z) - 1 - z) + z / 2 otherwise, with a+ = softplus(p) and a- = 1/2 + softplus(q) from the layer's two learned
    numbers ``act`` = (p, q); both are taken once at load, in 32-bit.  "relu2": act(z) = max(z, 0)^2, nothing learned."""

    @staticmethod
    def weight_shapes(spec):
        shapes = {"up": (spec.intermediate_size, spec.hidden_size), "down": (spec.hidden_size, spec.intermediate_size)}
        if spec.activation == "xielu":
            shapes["act"] = (2,)
        return shapes

    def __init__(self, spec, weights, runtime):
        if spec.activation not in ("xielu", "relu2"):
            raise ValueError(f"activation {spec.activation!r} is not built; 'xielu' and 'relu2' are")
        self.activation = spec.activation
        self.ops = runtime.ops
        self.w_up = self.ops.prepare_matrix(weights["up"])
        self.w_down = self.ops.prepare_matrix(weights["down"])
        if self.activation == "xielu":
            pq = torch.nn.functional.softplus(weights["act"].float().cpu())
            self.a_pos, self.a_neg = float(pq[0]), 0.5 + float(pq[1])

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h):
        if self.activation == "relu2":
            return self.ops.linear(self.ops.linear_relu2(h, self.w_up), self.w_down)
        return self.ops.linear(self.ops.linear_xielu(h, self.w_up, self.a_pos, self.a_neg), self.w_down)


register_part("ff", "gated_mlp", GatedMLP)
register_part("ff", "act_mlp", ActMLP)
