"""Rotary position encoding: the per-pair inverse frequencies, plain or llama3-scaled.

The reference takes its cos/sin tables from ``LlamaRotaryEmbedding`` for every position up to
max_position_embeddings and keeps them in float32 (tokasaurus/model/llama.py:559-570), then
gathers rows by position (llama.py:576-578) and applies ``apply_rotary_pos_emb`` (llama.py:243-256).
Those tables equal ``cos(pos * inv_freq)``, ``sin(pos * inv_freq)`` with the inverse frequencies
below, so this engine keeps only ``inv_freq`` (head_dim/2 floats) and forms the angle in the
kernel, in float32, as the same product.

    inv_freq_j = theta ** (-2j / rotary_dim),  j in [0, rotary_dim/2)
    llama3:  wavelen = 2*pi / inv_freq
             wavelen > orig/low_freq_factor   ->  inv_freq / factor
             wavelen < orig/high_freq_factor  ->  inv_freq
             otherwise  smooth = (orig/wavelen - low) / (high - low);
                        (1 - smooth) * inv_freq / factor + smooth * inv_freq
    yarn:    turns(t) = rotary_dim * ln(orig / (2 pi t)) / (2 ln theta)      (the pair index that makes t turns in orig positions)
             lo = max(floor(turns(fast)), 0),  hi = min(ceil(turns(slow)), rotary_dim - 1)
             ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)
             inv_freq_j / factor * ramp_j + inv_freq_j * (1 - ramp_j);   cos and sin times 0.1 ln(factor) + 1
"""

from __future__ import annotations

import math

import torch

from tokasaurus_b200.parts.base import PositionEncoding


class NoPositionEncoding(PositionEncoding):
    kind = "none"
    rotary_dim = 0

    def inv_freq(self) -> None:
        return None


class RotaryEncoding(PositionEncoding):
    kind = "rotary"

    def __init__(self, rotary_dim: int, theta: float, scaling_type: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 8192, yarn_fast: float = 32.0, yarn_slow: float = 1.0):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, got {rotary_dim}")
        if scaling_type not in ("default", "llama3", "yarn"):
            raise ValueError(f"unknown rotary scaling {scaling_type!r}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.scaling_type = scaling_type
        self.factor = float(factor)
        self.low_freq_factor = float(low_freq_factor)
        self.high_freq_factor = float(high_freq_factor)
        self.original_max_position_embeddings = int(original_max_position_embeddings)
        self.yarn_fast, self.yarn_slow = float(yarn_fast), float(yarn_slow)
        if scaling_type == "yarn" and not (self.factor > 0 and self.yarn_fast > 0 and self.yarn_slow > 0 and self.theta > 1):
            raise ValueError("yarn scaling needs a positive factor and turn counts, and a base above 1")

    def magnitude(self) -> float:
        """The factor on every cosine and sine (1 unless the scaling scheme has one)."""
        return 0.1 * math.log(self.factor) + 1.0 if self.scaling_type == "yarn" else 1.0

    def inv_freq64(self) -> torch.Tensor:
        """float64 [rotary_dim / 2] ``theta^(-2j / rotary_dim)``, on the CPU, for kernels that form their angles in
        float64 (plain frequencies, or yarn's blend of scaled and unscaled ones)."""
        if self.scaling_type not in ("default", "yarn"):
            raise ValueError("float64 frequencies exist for the plain and the yarn rotary encoding")
        d = self.rotary_dim
        f = self.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        if self.scaling_type == "default":
            return f
        orig = float(self.original_max_position_embeddings)

        def turns(t: float) -> float:
            return d * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(turns(self.yarn_fast)), 0)
        hi = min(math.ceil(turns(self.yarn_slow)), d - 1)
        ramp = ((torch.arange(d // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp)

    def inv_freq(self) -> torch.Tensor:
        """float32 [rotary_dim / 2], on the CPU."""
        d = self.rotary_dim
        if self.scaling_type == "yarn":
            return self.inv_freq64().to(torch.float32)
        inv = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d))
        if self.scaling_type == "default":
            return inv
        orig = self.original_max_position_embeddings
        low_wavelen = orig / self.low_freq_factor
        high_wavelen = orig / self.high_freq_factor
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > low_wavelen, inv / self.factor, inv)
        smooth = (orig / wavelen - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
        mid = (1 - smooth) * scaled / self.factor + smooth * scaled
        is_mid = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
        return torch.where(is_mid, mid, scaled).to(torch.float32)


class SinusoidalPositions(PositionEncoding):
    """A position vector added to the embedding: entry 2i is sin(p * base^(-2i / width)), entry 2i + 1 the cosine of
    the same angle.  Frequencies, angles, sines and cosines are float64 (the kernel forms the angle as the product of
    position and frequency); what is added to the float32 stream is their rounding."""

    kind = "additive"
    rotary_dim = 0

    def __init__(self, width: int, base: float = 10000.0):
        self.width = int(width)
        self.base = float(base)

    def inv_freq(self) -> torch.Tensor:
        """float64 [ceil(width / 2)], on the CPU."""
        i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
        return self.base ** (-2.0 * i / self.width)
