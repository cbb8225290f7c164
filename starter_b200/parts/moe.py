"""Mixture of experts (kind "moe"): a 32-bit router, gated experts, identity experts, a shared expert.

    s = softmax(W_r h) over experts + identity outputs        (32-bit; h is what the experts read)
    chosen = the ``top`` largest of s + correction;  weight_e = s_e / (sum of the chosen s + 1e-20) * route_scale
    y = sum over chosen e of weight_e * expert_e(h)  +  shared(h)

With ``over_chosen`` the ``top`` largest logits (+ bias, + correction when there is one) are chosen and weighted by
the softmax over the chosen logits alone; the experts' activation is the clamped one or silu(gate) * up.

An identity output stands for an expert that hands its input back: it adds weight * h and reads no matrix.  The
experts' matrices are kept stacked ([experts, 2 ff, width] gate over up, [experts, width, ff]) and the chosen
(token, expert) pairs are sorted by expert on the device, so that a step runs one grouped product per matrix whatever
the router chose and nothing is read back to the host.  The weighted sum over a token's experts, its identity share
and the shared expert's output meet in 32-bit in one kernel.
"""

from __future__ import annotations

import torch

from .registry import build_part, register_part


class MixtureOfExperts:
    @staticmethod
    def weight_shapes(spec):
        h, ff = spec.hidden_size, spec.expert.intermediate_size
        shapes = {"router": (spec.n_experts + spec.n_identity, h)}
        if spec.correction:
            shapes["correction"] = (spec.n_experts + spec.n_identity,)
        if spec.router_bias:
            shapes["router_bias"] = (spec.n_experts + spec.n_identity,)
        for e in range(spec.n_experts):
            shapes.update({f"e{e}_gate": (ff, h), f"e{e}_up": (ff, h), f"e{e}_down": (h, ff)})
        if spec.shared is not None:
            s = spec.shared.intermediate_size
            shapes.update({"shared_gate": (s, h), "shared_up": (s, h), "shared_down": (h, s)})
        return shapes

    def __init__(self, spec, weights, runtime):
        E, total = spec.n_experts, spec.n_experts + spec.n_identity
        if not 1 <= spec.top <= total:
            raise ValueError(f"{spec.top} of {total} experts cannot be chosen")
        if spec.expert.activation not in ("clamped_swish", "silu"):
            raise ValueError(f"experts with the activation {spec.expert.activation!r} are not built; 'clamped_swish' and 'silu' are")
        if spec.n_identity and spec.over_chosen:
            raise ValueError("identity outputs go with the softmax over all outputs")
        self.spec = spec
        self.ops = runtime.ops
        self.router = weights["router"].float().contiguous()                 # 32-bit logits
        self.correction = weights["correction"].float().contiguous() if spec.correction else None
        self.bias = weights["router_bias"].float().contiguous() if spec.router_bias else None
        # alpha None: silu(gate) * up; else the clamped activation with its sigmoid factor and limit
        self.alpha = float(spec.expert.alpha) if spec.expert.activation == "clamped_swish" else None
        self.limit = float(spec.expert.limit) if spec.expert.activation == "clamped_swish" else 0.0
        self.w_gate_up = torch.stack([torch.cat([weights[f"e{e}_gate"], weights[f"e{e}_up"]], dim=0) for e in range(E)]).contiguous() \
            if E else None
        self.w_down = torch.stack([weights[f"e{e}_down"] for e in range(E)]).contiguous() if E else None
        self.shared = None
        if spec.shared is not None:
            self.shared = build_part("ff", spec.shared, {r: weights["shared_" + r] for r in ("gate", "up", "down")}, runtime)

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h):
        s, ops = self.spec, self.ops
        base = self.shared.forward(ctx, h) if self.shared is not None else None
        chosen, weight = ops.moe_route(h, self.router, self.correction, s.top, float(s.route_scale), bias=self.bias,
                                       over_chosen=s.over_chosen)
        return ops.moe_experts(h, chosen, weight, self.w_gate_up, self.w_down, s.n_experts, self.alpha, self.limit, base)


register_part("ff", "moe", MixtureOfExperts)
