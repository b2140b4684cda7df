"""Rotary position encoding: the per-step cos/sin tables.

src/llm_pipeline/models/qwen3/custom_builder.py:269-288: ``inv_freq[j] = 1 / theta^(2j/d)``
(float32), angle = position * inv_freq, cos and sin of the angle times ``attention_scaling``
(1.0), all in float32. The tables are ``[tokens, rotary_dim / 2]`` because the reference's
``cat(freqs, freqs)`` repeats them; the mixer's kernel pairs entry j with j + rotary_dim/2
(custom_builder.py:85-99). The reference rounds the tables to the activations' type
(custom_builder.py:288); here they stay float32.

``frequency_scaling`` (optional: ``factor``, ``low``, ``high``, ``original``) rescales the frequencies by wavelength
before any angle is taken: with wavelength l = 2 pi / f, f stays where l < original / high, becomes f / factor where
l > original / low, and between the two is the blend (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
The frequencies are computed in float64 on the host and stored as float32; angles are float32 products.

A rule with ``"kind": "ramp"`` (``factor``, ``original``, ``fast``, ``slow``) blends by the entry's index instead: with
``where(t) = dims * ln(original / (2 pi t)) / (2 ln theta)`` (the index whose wave makes t turns over the original length),
lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
the frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``. A design that also scales cos and sin (by
``0.1 ln(factor) + 1``, say) passes that number as ``scaling``."""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..ops import kernels
from .base import PositionEncoding
from .registry import register_position


@register_position("rotary")
class RotaryPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str, rotary_dim: int, theta: float, scaling: float = 1.0,
                 frequency_scaling: Optional[Dict[str, float]] = None):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        self.prefix, self.rotary_dim, self.theta, self.scaling = prefix, int(rotary_dim), float(theta), float(scaling)
        self.frequency_scaling = dict(frequency_scaling) if frequency_scaling else None
        if self.frequency_scaling is None:
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float() / self.rotary_dim
            self._inv_freq_cpu = 1.0 / (self.theta ** exponent)
        else:
            rule = self.ramp_frequencies if self.frequency_scaling.get("kind") == "ramp" else self.rescaled_frequencies
            self._inv_freq_cpu = torch.tensor(rule(self.rotary_dim, self.theta, self.frequency_scaling), dtype=torch.float64).float()
        self._inv_freq = None

    @staticmethod
    def rescaled_frequencies(rotary_dim: int, theta: float, rule: Dict[str, float]):
        factor, low, high, original = (float(rule[k]) for k in ("factor", "low", "high", "original"))
        if not (factor > 0 and high > low and original > 0):
            raise ValueError(f"frequency scaling needs factor > 0, high > low and original > 0, got {rule}")
        out = []
        for j in range(rotary_dim // 2):
            f = theta ** (-2.0 * j / rotary_dim)
            wave = 2.0 * math.pi / f
            if wave < original / high:
                out.append(f)
            elif wave > original / low:
                out.append(f / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return out

    @staticmethod
    def ramp_frequencies(rotary_dim: int, theta: float, rule: Dict[str, float]):
        factor, original, fast, slow = (float(rule[k]) for k in ("factor", "original", "fast", "slow"))
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and theta > 1):
            raise ValueError(f"a frequency ramp needs positive factor, original, fast and slow, got {rule}")

        def where(turns: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(where(fast)), 0)
        hi = min(math.ceil(where(slow)), rotary_dim - 1)
        out = []
        for i in range(rotary_dim // 2):
            f = theta ** (-2.0 * i / rotary_dim)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return out

    def tables(self, ctx):
        if self._inv_freq is None or self._inv_freq.device != ctx.device:
            self._inv_freq = self._inv_freq_cpu.to(ctx.device)
        half = self.rotary_dim // 2
        cos = torch.empty((ctx.num_tokens, half), dtype=torch.float32, device=ctx.device)
        sin = torch.empty_like(cos)
        kernels.rope_tables(ctx.positions, self._inv_freq, self.scaling, cos, sin)
        return cos, sin
