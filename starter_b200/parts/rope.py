"""Rotary position encoding (kind "rope"), rotate-half pairing.

Tables as the reference builds them (engine/model.py:78-93): inv_freq in
32-bit, angle = position * inv_freq in 32-bit, cos and sin taken in 32-bit and
only then rounded to the run's dtype.  Columns d and d + D/2 share an angle,
so the table holds D/2 columns.
"""

from __future__ import annotations

import math

import torch

from .registry import register_part


class RotaryEmbedding:
    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        self.runtime = runtime
        self.cos = None
        self.sin = None

    def prepare(self, n_positions: int) -> None:
        """Build (or grow) the tables to cover positions 0..n_positions-1."""
        if self.cos is not None and self.cos.shape[0] >= n_positions:
            return
        d = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        positions = torch.arange(n_positions, dtype=torch.float32)
        angles = positions[:, None] * inv_freq[None, :]
        rt = self.runtime
        self.cos = angles.cos().to(rt.dtype).to(rt.device).contiguous()
        self.sin = angles.sin().to(rt.dtype).to(rt.device).contiguous()

    def fused_rotary(self):
        """(cos, sin, rotary_dim) for the kernel that norms, rotates and stores in one pass."""
        return self.cos, self.sin, self.rotary_dim


class PairRotary:
    """Kind "rope_pairs": neighbouring columns (2j, 2j + 1) turn together.  It keeps no table of sines: the kernels
    that rotate take the row's position from the step's batch, multiply it in 32-bit with the frequency
    theta**(-2j / rotary_dim) from ``frequencies`` (32-bit, [rotary_dim / 2]) and take sine and cosine there."""

    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.theta = float(spec.theta)
        self.rotary_dim = int(spec.rotary_dim)
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
        self.frequencies = (torch.tensor(self.theta, dtype=torch.float32) ** (-2.0 * j / self.rotary_dim)).to(runtime.device)

    def prepare(self, n_positions: int) -> None:
        pass


class ScaledHalfRotary:
    """Kind "rope_half_scaled": column i of the first ``rotary_dim`` turns with column i + rotary_dim/2; frequencies
    stretched by wavelength when the spec gives a factor (see ScaledHalfRopeSpec).  No table: ``half_rotary`` hands the
    kernels 32-bit frequencies, and they take angle = position * frequency, sine and cosine in 32-bit."""

    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        dims = int(spec.rotary_dim)
        if dims <= 0 or dims % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.rotary_dim = dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = float(spec.theta) ** (-2.0 * i / dims)
        self.magnitude = 1.0
        if spec.factor is not None:
            def pair_at(turns):
                return dims * math.log(float(spec.original) / (2.0 * math.pi * float(turns))) / (2.0 * math.log(float(spec.theta)))
            lo = max(math.floor(pair_at(spec.fast)), 0)
            hi = min(math.ceil(pair_at(spec.slow)), dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / float(spec.factor) * ramp + f * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(float(spec.factor)) + 1.0
        self.frequencies = f.to(torch.float32).to(runtime.device)

    def prepare(self, n_positions: int) -> None:
        pass

    def half_rotary(self):
        """(frequencies [rotary_dim / 2] 32-bit, rotary_dim, what multiplies cosines and sines)."""
        return self.frequencies, self.rotary_dim, self.magnitude


class SinusoidEmbedding:
    """Kind "sinusoid": a position vector added to the embedded rows, column 2i = sin(p * base**(-2i / size)), column
    2i + 1 = cos of the same angle.  It enters at the embedding: ``embed`` makes the first residual, 32-bit, from the
    token ids and the rows' positions (angle = position * frequency in the kernel, 32-bit frequencies, no table)."""

    @staticmethod
    def weight_shapes(spec):
        return {}

    def __init__(self, spec, weights, runtime):
        if spec.size < 1:
            raise ValueError(f"a position vector has at least one column, got {spec.size}")
        self.size = int(spec.size)
        i = torch.arange((self.size + 1) // 2, dtype=torch.float64)
        self.frequencies = (float(spec.base) ** (-2.0 * i / self.size)).to(torch.float32).to(runtime.device)
        self.ops = runtime.ops

    def prepare(self, n_positions: int) -> None:
        pass

    def embed(self, ctx, tokens, table):
        return self.ops.embed_sinusoid(ctx, tokens, table, self.frequencies)


register_part("position", "sinusoid", SinusoidEmbedding)
register_part("position", "rope", RotaryEmbedding)
register_part("position", "rope_half_scaled", ScaledHalfRotary)
register_part("position", "rope_pairs", PairRotary)
