"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32, the scale multiplied after
the normalisation and not as (1 + w) (reference: src/layer/normalization.cpp:10-18,
deps/ttl/src/kernels/normalization/normalization.cu:76-139).

LayerNorm: mean and variance of the row, a scale and (where the spec names one) a shift."""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import NormSpec
from ..kernels import ops
from ..weights.loader import ROLE_NORM, ROLE_ZERO, WeightDecl
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec: NormSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.dtype = dtype
        self.weight = weights[spec.weight]
        self._scale32 = self.weight.float().contiguous()     # what the fused residual form reads

    @staticmethod
    def weight_decls(spec: NormSpec) -> dict[str, WeightDecl]:
        return {spec.weight: WeightDecl((spec.size,), ROLE_NORM)}

    def weights_read(self) -> list[torch.Tensor]:
        return [self.weight]          # (the float32 copy of the scales stands in for them, not beside them)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype == torch.float32 and self.dtype != torch.float32:
            return ops.sum_rms_norm(x, None, None, self.weight, self.eps, out_dtype=self.dtype)    # a float32 stream
        return ops.rmsnorm(x, self.weight, self.eps)

    def sum_forward(self, stream: torch.Tensor, summands: tuple) -> torch.Tensor:
        """stream (float32) += (the summands added to each other), in place and in float32; returns the norm
        of the sum in the model's type.  A summand is [rows, H], or a float32 [H] shift that goes on every
        row.  Two summands and a shift take one kernel for the sums and the norm."""
        rows = [s for s in summands if s.dim() == 2]
        shifts = [s for s in summands if s.dim() == 1]
        for more in rows[2:]:
            stream.add_(more)
        shift = None
        if shifts and rows:
            shift = shifts[0] if len(shifts) == 1 else torch.stack(shifts).sum(0)
        elif shifts:
            stream.add_(torch.stack(shifts).sum(0))
        a = rows[0] if len(rows) > 0 else None
        b = rows[1] if len(rows) > 1 else None
        return ops.sum_rms_norm(stream, a, b, self.weight, self.eps, out_dtype=self.dtype, bias=shift)

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps)

    def add_scaled(self, residual: torch.Tensor, delta: torch.Tensor, mult: float,
                   then: "RMSNorm | None" = None, rounded_sum: bool = False) -> torch.Tensor | None:
        """residual (float32) += mult * norm(delta), in place and in one kernel; with ``then`` also returns
        then(residual), with ``rounded_sum`` the sum itself in delta's type: the form a block with norms
        behind its parts uses."""
        if then is None:
            return ops.residual_rms_norm(residual, delta, self._scale32, self.eps, mult, rounded_sum=rounded_sum)
        return ops.residual_rms_norm(residual, delta, self._scale32, self.eps, mult, then._scale32, then.eps)

    def as_rms_scale(self) -> tuple[torch.Tensor, float]:
        return self.weight, self.eps


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b, the variance being the mean of the squared deviations;
    statistics, scale and shift in float32.  The input may be a float32 residual stream or a tensor of
    the model's type; the output has the model's type.  ``add_scaled`` is the fused form a block with
    norms behind its parts uses: residual += m * this_norm(delta), then the next norm of the sum."""

    graph_safe = True

    def __init__(self, spec: NormSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.dtype = dtype
        self.weight = weights[spec.weight].float().contiguous()
        self.bias = weights[spec.bias].float().contiguous() if spec.bias is not None else None

    @staticmethod
    def weight_decls(spec: NormSpec) -> dict[str, WeightDecl]:
        decls = {spec.weight: WeightDecl((spec.size,), ROLE_NORM)}
        if spec.bias is not None:           # a spec without the name of a shift: scale only
            decls[spec.bias] = WeightDecl((spec.size,), ROLE_ZERO)
        return decls

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps, out_dtype=self.dtype)

    def add_scaled(self, residual: torch.Tensor, delta: torch.Tensor, mult: float,
                   then: "LayerNorm | None" = None, rounded_sum: bool = False) -> torch.Tensor | None:
        """residual (float32) += mult * norm(delta), in place; with ``then`` also returns then(residual),
        with ``rounded_sum`` the sum itself in delta's type."""
        if then is None:
            return ops.residual_layer_norm(residual, delta, self.weight, self.bias, self.eps, mult,
                                           rounded_sum=rounded_sum)
        return ops.residual_layer_norm(residual, delta, self.weight, self.bias, self.eps, mult,
                                       then.weight, then.bias, then.eps)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
