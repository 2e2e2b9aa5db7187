"""Rotary position encoding: pair ``i`` of a head's first ``rot_dim`` values turns by
``pos * theta^(-2i/rot_dim)``.  Pairing ``half`` (NEOX) pairs value ``i`` with ``i + rot_dim/2``
(crates/bfi-core/src/cpu.rs:650-670; qwen3 uses the whole head, no frequency scaling:
crates/bfi-models/src/qwen3.rs:150-163); pairing ``adjacent`` pairs value ``2i`` with ``2i + 1``.

Frequency scaling ``yarn`` (parameters factor, original, fast, slow) slows the low frequencies
down by ``factor`` and leaves the high ones alone, with a linear ramp between: with
``dim(t) = rot_dim * ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(dim(fast)), 0)``,
``hi = min(ceil(dim(slow)), rot_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``
the frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cos and sin are both
multiplied by ``0.1 * ln(factor) + 1``.

The angles are evaluated in float64 on the host, once, and the table of (cos, sin) is rounded to
float32: it is at least as exact as evaluating ``pos / theta^(2i/d)`` in float32 per token, which
is what the reference does.  The attention kernels read the table in the same pass as the q/k
norms and the cache write.
"""
from __future__ import annotations

import math

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def yarn_frequencies(inv_freq: torch.Tensor, theta: float, rot_dim: int, factor: float, original: float,
                     fast: float, slow: float):
    """The scaled frequencies (float64) and the factor on cos and sin."""
    def dim_of(turns: float) -> float:
        return rot_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), rot_dim - 1)
    i = torch.arange(inv_freq.numel(), dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return inv_freq / factor * ramp + inv_freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotary_table(theta: float, rot_dim: int, positions: int, device, scaling=None) -> torch.Tensor:
    """float32 ``[positions, rot_dim/2, 2]`` of (cos, sin)."""
    half = rot_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rot_dim)
    magnitude = 1.0
    if scaling is not None:
        inv_freq, magnitude = yarn_frequencies(inv_freq, float(theta), rot_dim, scaling["factor"], scaling["original"],
                                               scaling["fast"], scaling["slow"])
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    table = (torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1) * magnitude).to(torch.float32)
    return table.contiguous().to(device)


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, theta: float, rot_dim: int, pairing: str = "half", scaling=None):
        if rot_dim % 2 != 0 or rot_dim <= 0:
            raise ValueError(f"rotary width must be even and positive, got {rot_dim}")
        if pairing not in ("half", "adjacent"):
            raise ValueError(f"rotary pairing must be 'half' or 'adjacent', got {pairing!r}")
        self.theta = float(theta)
        self.rot_dim = int(rot_dim)
        self.pairing = pairing
        self.scaling = None
        if scaling is not None:
            scaling = dict(scaling)
            if scaling.pop("kind", "yarn") != "yarn":
                raise ValueError("rotary frequency scaling: only 'yarn' is known")
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in scaling]
            if missing:
                raise ValueError(f"yarn scaling lacks {missing}")
            self.scaling = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if self.scaling["factor"] <= 0 or self.scaling["original"] <= 0 or self.scaling["fast"] <= 0 \
                    or self.scaling["slow"] <= 0 or self.theta <= 1.0:
                raise ValueError("yarn scaling needs positive factor, original, fast, slow and a base above 1")
        self.table = None

    def prepare(self, runtime, max_positions: int) -> None:
        key = ("rotary", self.theta, self.rot_dim, max_positions,
               tuple(sorted(self.scaling.items())) if self.scaling else None)
        table = runtime.shared.get(key)
        if table is None:
            table = rotary_table(self.theta, self.rot_dim, max_positions, runtime.device, self.scaling)
            runtime.shared[key] = table
        self.table = table

    def fused_rotary(self):
        return self.table, self.rot_dim


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True

    def fused_rotary(self):
        return None, 0
