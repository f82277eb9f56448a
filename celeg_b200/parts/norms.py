"""Norm parts. Interface of a norm:

    Norm(params, weights, rt)
    add_norm(residual, delta, out, n_rows, rows=None)
        residual: float32 [T, width] (updated in place with ``delta`` when ``rows`` is None)
        delta:    activation-type [T, width] or None
        out:      activation-type [n_rows, width]
        rows:     int32 row list to gather (then the residual is left untouched)
    as_prologue() -> (weight, eps) or None      optional: a plain RMSNorm, which the runtime may split
                                                between the products before and after it
    adds_two = True                             optional: add_norm also takes ``delta_b``, a second output owed to
                                                the stream (blocks with mixer and feed-forward side by side)
    add_norm_pair(residual, delta, delta_b, other, out, other_out, n_rows)
                                                optional: this norm and ``other`` (same class) of the same rows in
                                                one pass, both deltas added for good
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime


@register_part("norm", "rmsnorm")
class RmsNorm:
    """y = x / sqrt(mean(x^2) + eps) * w, the weight a direct scale
    (celeg src/backend/cpu/kernels/elementwise.cpp:56-76). With ``weight_offset`` c the stored tensor lies around
    zero and stands for the scale c + w (the sum is made once, in float32, when the part is built)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], rt: Runtime):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = rt.vector(weights["weight"])
        offset = float(params.get("weight_offset", 0.0))
        if offset != 0.0:
            self.weight.add_(offset)
        if self.weight.shape != (self.width,):
            raise ValueError(f"rmsnorm weight has shape {tuple(self.weight.shape)}, expected ({self.width},)")

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor, n_rows: int,
                 rows: Optional[torch.Tensor] = None) -> None:
        kernels.add_rmsnorm(residual, delta, self.weight, out, self.eps, rows=rows, n_rows=n_rows)

    def as_prologue(self):
        return self.weight, self.eps


@register_part("norm", "dynamic_tanh")
class DynamicTanh:
    """y = tanh(alpha x) w + b with a scalar alpha: no mean, no variance, hence no reduction over the row
    (Zhu et al., "Transformers without Normalization", 2025). tanh and the affine part in float32."""

    adds_two = True

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], rt: Runtime):
        self.width = int(params["width"])
        self.weight = rt.vector(weights["weight"])
        self.bias = rt.vector(weights["bias"])
        self.alpha = float(weights["alpha"].to(torch.float32).reshape(-1)[0])
        for name, vector in (("weight", self.weight), ("bias", self.bias)):
            if vector.shape != (self.width,):
                raise ValueError(f"dynamic_tanh {name} has shape {tuple(vector.shape)}, expected ({self.width},)")

    def _terms(self, out: torch.Tensor):
        return self.weight, self.bias, self.alpha, out

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor, n_rows: int,
                 rows: Optional[torch.Tensor] = None, delta_b: Optional[torch.Tensor] = None) -> None:
        kernels.add_dyt(residual, delta, delta_b, n_rows, self._terms(out), rows=rows)

    def add_norm_pair(self, residual: torch.Tensor, delta: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                      other: "DynamicTanh", out: torch.Tensor, other_out: torch.Tensor, n_rows: int) -> None:
        kernels.add_dyt(residual, delta, delta_b, n_rows, self._terms(out), other._terms(other_out))


@register_part("norm", "layernorm")
class LayerNorm:
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w (+ b), var the mean of the squared deviations from the mean (Ba,
    Kiros and Hinton, "Layer Normalization", 2016); the tensor ``bias`` is optional. Sums in float32, two passes."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], rt: Runtime):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = rt.vector(weights["weight"])
        self.bias = rt.vector(weights["bias"]) if "bias" in weights else None
        for name, vector in (("weight", self.weight), ("bias", self.bias)):
            if vector is not None and vector.shape != (self.width,):
                raise ValueError(f"layernorm {name} has shape {tuple(vector.shape)}, expected ({self.width},)")

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor, n_rows: int,
                 rows: Optional[torch.Tensor] = None) -> None:
        kernels.add_layernorm(residual, delta, self.weight, out, self.eps, rows=rows, n_rows=n_rows, bias=self.bias)
