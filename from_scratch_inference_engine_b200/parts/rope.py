"""Rotary position encoding: a cos/sin table computed in 64-bit on the host."""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .base import Part, register_part


def rotary_table(theta: float, rotary_dim: int, length: int) -> np.ndarray:
    """[length, rotary_dim] float32: cos(pos * f_i) for i < rotary_dim/2, then sin.

    f_i = theta^(-2i/rotary_dim) and the angle are computed in 64-bit and rounded once,
    as the reference computes them per element (src/model/nn.cpp:122-137)."""
    half = rotary_dim // 2
    inv_freq = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / rotary_dim)
    angles = np.arange(length, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.concatenate([np.cos(angles), np.sin(angles)], axis=1).astype(np.float32)


def yarn_rotary_table(theta: float, rotary_dim: int, length: int, factor: float, original: float,
                      fast: float, slow: float) -> np.ndarray:
    """The table of `rotary_table` with YaRN's change of the frequencies and of the magnitude.

    With dim(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns by position * (f_i / factor * ramp_i + f_i * (1 - ramp_i)): pairs that turn often
    within the original length keep their frequency, slow ones are stretched by `factor`.  Cos and
    sin are both multiplied by 0.1 ln(factor) + 1.  64-bit on the host, rounded once."""
    import math
    half = rotary_dim // 2
    index = np.arange(half, dtype=np.float64)
    inv_freq = np.power(float(theta), -2.0 * index / rotary_dim)

    def dim_of(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), rotary_dim - 1)
    ramp = np.clip((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    inv_freq = inv_freq / factor * ramp + inv_freq * (1.0 - ramp)
    magnitude = 0.1 * math.log(factor) + 1.0
    angles = np.arange(length, dtype=np.float64)[:, None] * inv_freq[None, :]
    return (np.concatenate([np.cos(angles), np.sin(angles)], axis=1) * magnitude).astype(np.float32)


def llama3_rotary_table(theta: float, rotary_dim: int, length: int, factor: float, original: float,
                        low: float, high: float) -> np.ndarray:
    """The table of `rotary_table` with the frequencies rescaled by wavelength: with l = 2 pi / f_i,
    pair i keeps f_i where l < original / high, turns at f_i / factor where l > original / low, and
    in between, with t = (original / l - low) / (high - low), at (1 - t) f_i / factor + t f_i.
    64-bit on the host, rounded once."""
    import math
    half = rotary_dim // 2
    inv_freq = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / rotary_dim)
    wavelength = 2.0 * math.pi / inv_freq
    blend = (original / wavelength - low) / (high - low) if high != low else np.ones_like(inv_freq)
    mixed = (1.0 - blend) * inv_freq / factor + blend * inv_freq
    scaled = np.where(wavelength < original / high, inv_freq,
                      np.where(wavelength > original / low, inv_freq / factor, mixed))
    angles = np.arange(length, dtype=np.float64)[:, None] * scaled[None, :]
    return np.concatenate([np.cos(angles), np.sin(angles)], axis=1).astype(np.float32)


@register_part("position", "rotary")
class RotaryEncoding(Part):
    """Rotation of pairs over the first `rotary_dim` of each head: `pairing` "half" pairs
    dimension i with i + rotary_dim/2, "interleaved" pairs 2i with 2i + 1; pair i turns by
    position * theta^(-2i/rotary_dim) either way, so both read the same table.  The rotation
    itself runs inside the mixer's kernel; this part owns the table and names the pairing."""

    capturable = True

    def __init__(self, prefix: str, theta: float, rotary_dim: int, max_position: int = 0,
                 pairing: str = "half"):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError("pairing must be 'half' or 'interleaved'")
        self.pairing = pairing
        self.prefix, self.theta = prefix, float(theta)
        self.rotary_dim, self.max_position = int(rotary_dim), int(max_position)
        self.table: Optional[torch.Tensor] = None

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        # as long as the configuration says, and at least as long as the cache can hold
        length = max(self.max_position, runtime.max_positions, 1)
        if self.rotary_dim == 0:
            self.table = runtime.shared_table(("rotary-none",),
                                              lambda: torch.zeros((1, 0), dtype=torch.float32))
            return
        self.table = runtime.shared_table(
            ("rotary", self.theta, self.rotary_dim, length),
            lambda: torch.from_numpy(rotary_table(self.theta, self.rotary_dim, length)))


@register_part("position", "yarn_rotary")
class YarnRotaryEncoding(RotaryEncoding):
    """`rotary` with YaRN scaling (`yarn_rotary_table`): `factor`, the `original` length, and the
    numbers of turns `fast` and `slow` between which the frequencies go over from kept to
    stretched.  The kernels read the table as they read the plain one: the magnitude factor is in
    its cos and sin."""

    def __init__(self, prefix: str, theta: float, rotary_dim: int, factor: float, original: float,
                 fast: float, slow: float, max_position: int = 0, pairing: str = "half"):
        super().__init__(prefix, theta, rotary_dim, max_position, pairing)
        if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or theta <= 1:
            raise ValueError("yarn_rotary: factor, original, fast and slow must be positive, theta above 1")
        self.factor, self.original = float(factor), float(original)
        self.fast, self.slow = float(fast), float(slow)

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        length = max(self.max_position, runtime.max_positions, 1)
        if self.rotary_dim == 0:
            self.table = runtime.shared_table(("rotary-none",),
                                              lambda: torch.zeros((1, 0), dtype=torch.float32))
            return
        self.table = runtime.shared_table(
            ("yarn_rotary", self.theta, self.rotary_dim, length, self.factor, self.original, self.fast,
             self.slow),
            lambda: torch.from_numpy(yarn_rotary_table(self.theta, self.rotary_dim, length, self.factor,
                                                       self.original, self.fast, self.slow)))


@register_part("position", "llama3_rotary")
class Llama3RotaryEncoding(RotaryEncoding):
    """`rotary` with the frequencies rescaled by wavelength (`llama3_rotary_table`): `factor`, the
    `original` length and the `low` and `high` numbers of turns within it between which a pair goes
    over from stretched to kept.  The kernels read the table as they read the plain one."""

    def __init__(self, prefix: str, theta: float, rotary_dim: int, factor: float, original: float,
                 low: float, high: float, max_position: int = 0, pairing: str = "half"):
        super().__init__(prefix, theta, rotary_dim, max_position, pairing)
        if factor <= 0 or original <= 0 or low <= 0 or high <= 0 or theta <= 1:
            raise ValueError("llama3_rotary: factor, original, low and high must be positive, theta above 1")
        self.factor, self.original = float(factor), float(original)
        self.low, self.high = float(low), float(high)

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        length = max(self.max_position, runtime.max_positions, 1)
        if self.rotary_dim == 0:
            self.table = runtime.shared_table(("rotary-none",),
                                              lambda: torch.zeros((1, 0), dtype=torch.float32))
            return
        self.table = runtime.shared_table(
            ("llama3_rotary", self.theta, self.rotary_dim, length, self.factor, self.original, self.low,
             self.high),
            lambda: torch.from_numpy(llama3_rotary_table(self.theta, self.rotary_dim, length, self.factor,
                                                         self.original, self.low, self.high)))


@register_part("position", "none")
class NoPositionEncoding(Part):
    """No position encoding: queries and keys are used as projected."""

    capturable = True

    rotary_dim = 0

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.table = None

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.table = runtime.shared_table(("rotary-none",),
                                          lambda: torch.zeros((1, 0), dtype=torch.float32))
