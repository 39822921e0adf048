"""Rotary position encoding of the `default` type (engine/model.py:126-161).

inv_freq[i] = 1 / theta^(2i/d) is computed in float32 from an integer range, exactly
as the reference does (engine/model.py:132-135); the angle position x inv_freq and its
cosine and sine are float32 on the device, one table per step shared by every layer
that uses the same (head_dim, theta). Pairs are (j, j + d/2) (engine/model.py:126-129).
"""

from __future__ import annotations

import math

import torch

from .base import POSITION_ENCODINGS, Part


@POSITION_ENCODINGS.register("rotary")
class Rotary(Part):
    """params: head_dim, theta. No tensors."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        if self.head_dim % 2:
            raise ValueError(f"rotary: head_dim {self.head_dim} must be even")
        exponent = torch.arange(0, self.head_dim, 2, dtype=torch.int64).to(torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (exponent / self.head_dim))).to(runtime.device)
        self._key = ("rotary", self.head_dim, self.theta)

    def table(self, ctx):
        """float32 [tokens, head_dim]: cosines in the first half of a row, sines in the second."""
        if self._key not in ctx.memo:
            ctx.memo[self._key] = self.ops.rotary_table(ctx.positions, self.inv_freq)
        return ctx.memo[self._key]


def banded_frequencies(freqs, factor: float, low: float, high: float, original: float):
    """Frequencies whose wavelength is short (below original / high) stay, long ones (above
    original / low) are divided by `factor`, and those between are blended linearly in
    original / wavelength."""
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            # high == low leaves no band between the two: a wavelength on the one border is kept
            s = (original / wavelength - low) / (high - low) if high != low else 1.0
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramped_frequencies(freqs, dims: int, base: float, factor: float, original: float, fast: float, slow: float):
    """(frequencies, amplitude) of the ramped scaling: pair i is divided by `factor` to the degree
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), where lo and hi are the pairs that turn
    `fast` and `slow` times within `original` positions (rounded down and up, kept inside the
    head); cosines and sines are multiplied by 0.1 ln(factor) + 1."""
    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("scaled_rotary")
class ScaledRotary(Part):
    """Cosines and sines for a rotated span of `dims` channels, with the frequencies base^(-2i/dims)
    rescaled for sequences longer than the ones the frequencies were made for. params: dims, base,
    scaling: None, or {"kind": "banded", factor, low, high, original}, or {"kind": "ramped",
    factor, original, fast, slow}. No tensors. The frequencies are worked out in double
    precision and rounded once to float32; the angle is a float32 product on the device. Which
    channels the span covers and how they pair is the mixer's business."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.dims = int(p["dims"])
        self.base = float(p["base"])
        if self.dims < 2 or self.dims % 2:
            raise ValueError(f"scaled_rotary: {self.dims} rotated channels are not pairs")
        freqs = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        self.amplitude = 1.0
        scaling = p.get("scaling")
        if scaling is not None:
            s = {k: float(v) for k, v in scaling.items() if k != "kind"}
            if scaling.get("kind") == "banded":
                freqs = banded_frequencies(freqs, s["factor"], s["low"], s["high"], s["original"])
            elif scaling.get("kind") == "ramped":
                freqs, self.amplitude = ramped_frequencies(freqs, self.dims, self.base, s["factor"], s["original"], s["fast"], s["slow"])
            else:
                raise ValueError(f"scaled_rotary: scaling kind {scaling.get('kind')!r} (banded, ramped)")
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self._key = ("scaled_rotary", self.dims, self.base, tuple(sorted((scaling or {}).items())))

    def table(self, ctx):
        """float32 [tokens, dims]: amplitude x cosines in the first half of a row, amplitude x sines in the second."""
        if self._key not in ctx.memo:
            ctx.memo[self._key] = self.ops.rotary_table(ctx.positions, self.inv_freq, self.amplitude)
        return ctx.memo[self._key]
