"""Rotary position encoding: pair i of rotary_dim/2 turns by position * theta^(-2i/rotary_dim),
rotate-half pairing (i, i + rotary_dim/2); angles in float32 (atomserve/model.py:142-185).
Dimensions beyond rotary_dim pass through unrotated (rotary_dim = head_dim for Qwen3).
`pairing="interleaved"` pairs neighbours (2i, 2i + 1) instead, with the same frequencies; the
mixers whose fused kernels know that pairing apply it (latent attention)."""

from __future__ import annotations

import math

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FusedRotary, PositionEncoding, register_part


class Rotary(PositionEncoding):
    def __init__(self, hidden_size: int, prefix: str, head_dim: int, theta: float, rotary_dim: int | None = None,
                 pairing: str = "half"):  # fmt: skip
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing {pairing!r} is neither 'half' nor 'interleaved'")
        self.pairing = pairing
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim  # (0: nothing turns)
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def prepare(self, device: torch.device) -> None:
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta**exponents)).to(device)

    def fused_rotary(self) -> FusedRotary:
        return FusedRotary(self.inv_freq, self.rotary_dim, self.pairing)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotate x [T, heads, head_dim] by its tokens' positions (the encoding on its own)."""
        if self.pairing != "half":
            raise NotImplementedError("the stand-alone rotary kernel pairs (i, i + rotary_dim / 2) only")
        return ops.rotary(x, positions, self.inv_freq, self.rotary_dim)


class ScaledRotary(Rotary):
    """Rotary encoding whose frequencies are stretched for contexts longer than the `original` one
    (the scheme known as YaRN). With f_i = theta^(-2i / rotary_dim): index(t) = rotary_dim
    ln(original / (2 pi t)) / (2 ln theta) is where a frequency makes t turns over the original
    context; lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), rotary_dim - 1),
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency becomes
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cosines and sines are multiplied by
    0.1 ln(factor) + 1 (`FusedRotary.magnitude`)."""

    def __init__(self, hidden_size: int, prefix: str, head_dim: int, theta: float, factor: float, original: float,
                 fast: float, slow: float, rotary_dim: int | None = None, pairing: str = "half"):  # fmt: skip
        super().__init__(hidden_size, prefix, head_dim, theta, rotary_dim, pairing)
        if not factor > 0 or not original > 0 or not fast > 0 or not slow > 0:
            raise ValueError("a scaled rotary encoding needs positive factor, original, fast and slow")
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        self.magnitude = 0.1 * math.log(self.factor) + 1.0

    def prepare(self, device: torch.device) -> None:
        dims = self.rotary_dim
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = self.theta ** (-2.0 * i / dims) if dims else i

        def index(turns: float) -> float:
            return dims * math.log(self.original / (2 * math.pi * turns)) / (2 * math.log(self.theta))

        if dims:
            lo, hi = max(math.floor(index(self.fast)), 0), min(math.ceil(index(self.slow)), dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / self.factor * ramp + f * (1.0 - ramp)
        self.inv_freq = f.to(torch.float32).to(device)

    def fused_rotary(self) -> FusedRotary:
        return FusedRotary(self.inv_freq, self.rotary_dim, self.pairing, self.magnitude)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("the stand-alone rotary kernel has no magnitude; mixers apply this encoding fused")


class BandScaledRotary(Rotary):
    """Rotary encoding whose slow frequencies are divided by `factor` for contexts longer than the
    `original` one, chosen by wavelength l_i = 2 pi / f_i: a wave shorter than original / high
    keeps f_i, one longer than original / low turns at f_i / factor, and between the two the
    frequencies are mixed, (1 - s) f_i / factor + s f_i with s = (original / l_i - low) /
    (high - low). Cosines and sines keep their size. The table is made once, in float64."""

    def __init__(self, hidden_size: int, prefix: str, head_dim: int, theta: float, factor: float, original: float,
                 low: float, high: float, rotary_dim: int | None = None, pairing: str = "half"):  # fmt: skip
        super().__init__(hidden_size, prefix, head_dim, theta, rotary_dim, pairing)
        if not factor > 0 or not original > 0 or not high > low >= 0:
            raise ValueError("a band-scaled rotary encoding needs factor > 0, original > 0 and high > low >= 0")
        self.factor, self.original, self.low, self.high = float(factor), float(original), float(low), float(high)

    def prepare(self, device: torch.device) -> None:
        dims = self.rotary_dim
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = self.theta ** (-2.0 * i / dims) if dims else i
        if dims:
            turns = self.original * f / (2.0 * math.pi)  # original / wavelength
            mix = torch.clamp((turns - self.low) / (self.high - self.low), 0.0, 1.0)
            mixed = (1.0 - mix) * f / self.factor + mix * f
            f = torch.where(turns > self.high, f, torch.where(turns < self.low, f / self.factor, mixed))
        self.inv_freq = f.to(torch.float32).to(device)


register_part("position", "band_scaled_rotary", BandScaledRotary)
register_part("position", "rotary", Rotary)
register_part("position", "scaled_rotary", ScaledRotary)
