"""Position-encoding parts. Interface:

    Position(params, rt)
    fused() -> dict or None      tables for the fused q/k kernel: {"inv_freq": float32 [rotary/2],
                                 "rotary_dim": int}; None means the mixer must call apply()
    apply(q, k, positions, tokens)   in-place encoding of q [T, Hq, d] and k [T, Hkv, d] views

Keys are cached after encoding, so an encoding must be a pure function of the absolute position.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from .registry import register_part
from .runtime import Runtime


@register_part("position", "rope_split_half")
class SplitHalfRope:
    """Rotary embedding over pairs (i, i + rotary/2): angle = position * theta^(-2i/rotary).
    Frequencies are computed in double and rounded to float32, the angle product and
    sin/cos are float32, as celeg's CPU kernel does (src/backend/cpu/kernels/rope.cpp:74-79;
    include/celeg/model/position.hpp:77-78). ``wavelength_scaling`` = {factor, low, high, original}
    rescales the frequencies (:func:`scale_by_wavelength`); ``linear_factor`` divides every frequency by a constant
    (positions counted in units of that many tokens)."""

    def __init__(self, params: Mapping, rt: Runtime):
        self.theta = float(params["theta"])
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        half = self.rotary_dim // 2
        exponents = torch.arange(half, dtype=torch.float64) * (-2.0 / self.rotary_dim)
        frequencies = torch.pow(torch.tensor(self.theta, dtype=torch.float64), exponents)
        scaling = params.get("wavelength_scaling")
        if scaling:
            frequencies = scale_by_wavelength(frequencies, float(scaling["factor"]), float(scaling["low"]),
                                              float(scaling["high"]), float(scaling["original"]))
        linear = params.get("linear_factor")
        if linear is not None:
            if float(linear) <= 0:
                raise ValueError(f"linear_factor {linear} must be positive")
            frequencies = frequencies / float(linear)
        self.inv_freq = frequencies.to(torch.float32).to(rt.device)

    def fused(self) -> Optional[dict]:
        return {"inv_freq": self.inv_freq, "rotary_dim": self.rotary_dim}


def scale_by_wavelength(frequencies: torch.Tensor, factor: float, low: float, high: float,
                        original: float) -> torch.Tensor:
    """Context extension by wavelength (the rule Llama 3.1 checkpoints state in ``rope_scaling``): a frequency
    whose wavelength 2 pi / f is shorter than original / high stays, one longer than original / low is divided
    by ``factor``, and between the two the frequency is (1 - s) f / factor + s f with
    s = (original / wavelength - low) / (high - low). In double, like the frequencies themselves."""
    if factor <= 0 or high <= low or original <= 0:
        raise ValueError("wavelength scaling needs factor > 0, high > low and original > 0")
    wavelength = 2.0 * math.pi / frequencies
    smooth = (original / wavelength - low) / (high - low)
    blended = (1.0 - smooth) * frequencies / factor + smooth * frequencies
    return torch.where(wavelength < original / high, frequencies,
                       torch.where(wavelength > original / low, frequencies / factor, blended))


@register_part("position", "rope_interleaved")
class InterleavedRope:
    """Rotary embedding over neighbouring pairs (2i, 2i + 1) of the first ``rotary_dim`` dimensions: angle =
    position * f_i, f_i = theta^(-2i/rotary_dim). ``yarn`` = {factor, original, fast, slow} rescales the
    frequencies by how many turns a wave makes over the original length (:func:`scale_by_turns`) and multiplies
    cos and sin by 0.1 ln(factor) + 1 (Peng et al., "YaRN: Efficient Context Window Extension of Large Language
    Models", 2023). Frequencies in double, rounded to float32; the angle product and sin/cos are float32 in the
    kernels. Mixers take it through ``fused()``: {"inv_freq", "rotary_dim", "interleaved": True, "magnitude"}."""

    def __init__(self, params: Mapping, rt: Runtime):
        self.theta = float(params["theta"])
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        exponents = torch.arange(self.rotary_dim // 2, dtype=torch.float64) * (-2.0 / self.rotary_dim)
        frequencies = torch.pow(torch.tensor(self.theta, dtype=torch.float64), exponents)
        self.magnitude = 1.0
        yarn = params.get("yarn")
        if yarn:
            frequencies = scale_by_turns(frequencies, self.theta, self.rotary_dim, float(yarn["factor"]),
                                         float(yarn["original"]), float(yarn["fast"]), float(yarn["slow"]))
            self.magnitude = 0.1 * math.log(float(yarn["factor"])) + 1.0
        self.inv_freq = frequencies.to(torch.float32).to(rt.device)

    def fused(self) -> Optional[dict]:
        return {"inv_freq": self.inv_freq, "rotary_dim": self.rotary_dim, "interleaved": True,
                "magnitude": self.magnitude}


def scale_by_turns(frequencies: torch.Tensor, theta: float, dims: int, factor: float, original: float, fast: float,
                   slow: float) -> torch.Tensor:
    """YaRN's rule. The (fractional) pair index at which a wave makes ``turns`` turns over ``original`` positions is
    d(turns) = dims ln(original / (2 pi turns)) / (2 ln theta). Pairs below lo = max(floor(d(fast)), 0) keep their
    frequency, pairs above hi = min(ceil(d(slow)), dims - 1) have it divided by ``factor``, and between the two the
    share of the divided frequency rises linearly: ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i). In double, like the frequencies themselves."""
    if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or theta <= 1:
        raise ValueError("scaling by turns needs factor, original, fast, slow > 0 and theta > 1")

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    pair = torch.arange(frequencies.shape[0], dtype=torch.float64)
    ramp = torch.clamp((pair - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return frequencies / factor * ramp + frequencies * (1.0 - ramp)


@register_part("position", "none")
class NoPosition:
    def __init__(self, params: Mapping, rt: Runtime):
        pass

    def fused(self) -> Optional[dict]:
        return {"inv_freq": None, "rotary_dim": 0}
