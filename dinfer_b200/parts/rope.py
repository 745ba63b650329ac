"""Rotary position encoding: pairs ``(i, i + rot/2)`` (neox) or ``(2i, 2i + 1)`` (interleaved), over the whole head
or its first ``rotary_dim`` elements, positions optionally divided by a factor (linear scaling).

A position encoding is a helper of a mixer.  Interface:
  ``fused_table()`` -> the ``[max_positions, rot]`` f32 table ``cos | sin`` when the rotation can be
                      done inside the q/k post-processing kernel, else None;
  ``apply(q, k, ctx)`` -> for encodings that are not a table rotation: change the ``[T, heads, D]``
                      views of q and k in place (called between the head norm and the cache write).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_TABLES: Dict[Tuple, torch.Tensor] = {}


def ramp_frequencies(rotary_dim: int, theta: float, factor: float, original: float, fast: float, slow: float):
    """(frequencies [rot / 2] in 64-bit, the factor on cos and sin) of a rotation stretched to ``factor`` times the
    ``original`` length by a ramp over the frequencies: with ``turn(t) = rot ln(original / (2 pi t)) / (2 ln theta)``
    the index at which a frequency makes t turns over the original length, frequencies below index ``lo =
    floor(turn(fast))`` stay, those above ``hi = ceil(turn(slow))`` are divided by ``factor``, and between the two the
    share ``(i - lo) / (hi - lo)`` of the divided one is mixed in.  cos and sin are multiplied by ``0.1 ln(factor) + 1``."""
    import math
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / rotary_dim)

    def turn(t: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo = max(math.floor(turn(fast)), 0)
    hi = min(math.ceil(turn(slow)), rotary_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / float(factor) * ramp + f * (1.0 - ramp), 0.1 * math.log(float(factor)) + 1.0


def rope_table(rotary_dim: int, theta: float, max_positions: int, device, scaling_factor: float = 1.0,
               ramp=None) -> torch.Tensor:
    """``[p, i] = cos(p f_i)``, ``[p, rot/2 + i] = sin(p f_i)``, ``f_i = theta^(-2i/rot) / scaling_factor``: angles in
    64-bit, stored in 32-bit (crates/layers/src/nn.rs:157-173).  ``ramp`` = (factor, original, fast, slow): the
    frequencies and the factor on cos and sin of ``ramp_frequencies`` instead."""
    key = (rotary_dim, float(theta), max_positions, str(device), float(scaling_factor), tuple(ramp) if ramp else None)
    t = _TABLES.get(key)
    if t is None:
        half = rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        mult = 1.0
        if ramp:
            inv_freq, mult = ramp_frequencies(rotary_dim, theta, *ramp)
        else:
            inv_freq = 1.0 / (float(theta) ** (2.0 * i / rotary_dim)) / float(scaling_factor)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        t = (torch.cat([ang.cos(), ang.sin()], dim=1) * mult).to(torch.float32).to(device).contiguous()
        _TABLES[key] = t
    return t


@POSITION_ENCODINGS.register("rope")
@POSITION_ENCODINGS.register("rope_neox")
class RotaryNeox(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``max_positions``, optional ``rotary_dim`` (default: the whole head),
    ``style`` ("neox", the default: element i turns with i + rot/2; "interleaved": element 2i with 2i + 1) and
    ``scaling_factor`` (positions divided by it; default 1), ``ramp`` (a dict ``factor``, ``original``, ``fast``,
    ``slow``: the stretched frequencies of ``ramp_frequencies``).  All of it is the table and one flag of the q/k kernel."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        # the table has a row per position the engine can reach (the model's own limit may be far beyond that)
        self.max_positions = min(int(params["max_positions"]), int(env.max_positions))
        style = params.get("style", "neox")
        if style not in ("neox", "interleaved"):
            raise ValueError(f"rotary style {style!r}: neox or interleaved")
        self.interleaved = style == "interleaved"
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        if not self.scaling_factor > 0:
            raise ValueError("scaling_factor must be positive")
        r = params.get("ramp")
        self.ramp = None if not r else (float(r["factor"]), float(r["original"]), float(r["fast"]), float(r["slow"]))
        if self.ramp and (self.scaling_factor != 1.0 or not (self.ramp[0] > 0 and self.ramp[1] > 0 and self.ramp[2] > 0 and self.ramp[3] > 0)):
            raise ValueError("ramp: positive factor, original, fast and slow, and no scaling_factor beside it")
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self._table: Optional[torch.Tensor] = None

    fused = True

    def fused_table(self) -> Optional[torch.Tensor]:
        if self._table is None:
            self._table = rope_table(self.rotary_dim, self.theta, self.max_positions, self.env.device,
                                     self.scaling_factor, self.ramp)
        return self._table

    def apply(self, q, k, ctx) -> None:       # the rotation is always fused
        raise NotImplementedError


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    fused = True

    def fused_table(self):
        return None

    def apply(self, q, k, ctx) -> None:
        return None
