"""Layer norm with a gain and (unless the spec says there is none) a bias: (x - mean) / sqrt(variance + eps) * weight + bias, the variance being
the mean of the squared deviations from the mean; all of it in float32 on the float32 residual stream.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .registry import register_part


class LayerNorm(Part):
    foldable = False  # no product carries this norm in its prologue or epilogue: it always runs as its own kernel

    def parameters(self):
        n = self.spec.weights
        out = [ParamRequest(n["weight"], (self.spec.size,), "gain")]
        return out + [ParamRequest(n["bias"], (self.spec.size,), "bias")] if getattr(self.spec, "bias", True) else out

    def load(self, tensors):
        n = self.spec.weights
        self.weight = self.runtime.vector(tensors[n["weight"]])
        self.bias = self.runtime.vector(tensors[n["bias"]]) if getattr(self.spec, "bias", True) else None

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                write_x: bool = True) -> torch.Tensor:
        """x += delta (if any; the stream then holds the sum, also when only some `rows` are normalised),
        then the norm of x, or of the rows of x that `rows` picks."""
        if delta is not None:
            ops.residual_add(x, delta)
        return ops.layernorm(x, self.weight, self.bias, self.spec.eps, self.runtime.compute_dtype, rows)


register_part("norm", "layernorm", LayerNorm)
