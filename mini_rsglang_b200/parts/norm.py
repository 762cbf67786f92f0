"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, statistics in float32
(reference: crates/kernels/src/ops.cu:66-78).  The weight multiplies plainly (no 1 + w).
LayerNorm: y = (x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import WeightSpec
from .base import NORMS, Norm, Normed, Prenormed


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    rides_on_products = True

    def __init__(self, prefix: str, width: int, eps: float, leaf: str = "weight"):
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)
        self.leaf = leaf                   # the weights' name below the part's root ("": the root itself)
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf), (self.width,), "vector")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.name(self.leaf)]

    def forward(self, x):
        out = torch.empty_like(x)
        kernels.rmsnorm(x, self.weight, self.eps, out)
        return out

    def add_norm(self, residual, delta, rows=None, write_back=True):
        if isinstance(delta, Prenormed):          # the stream holds the sum already
            if delta.norm is self and rows is None:
                return delta                      # and the product after this norm finishes it
            delta = None
        if isinstance(delta, Normed):             # the stream holds the sum, and this norm of it may be there already
            if delta.norm is self and rows is None:
                return delta.rows
            delta = None
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=self.runtime.dtype, device=residual.device)
        kernels.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows, write_back)
        return out


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """Layer norm with weight and bias, statistics in float32.  `leaf` and `bias_leaf` name the two tensors below the
    part's root ("": the root itself)."""

    def __init__(self, prefix: str, width: int, eps: float, leaf: str = "weight", bias_leaf: str = "bias"):
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)
        self.leaf, self.bias_leaf = leaf, bias_leaf
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf), (self.width,), "vector"), WeightSpec(self.name(self.bias_leaf), (self.width,), "bias")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight, self.bias = tensors[self.name(self.leaf)], tensors[self.name(self.bias_leaf)]

    def forward(self, x):
        """Rows of the engine's dtype, normed (no residual)."""
        out = torch.empty_like(x)
        kernels.add_layernorm(x.float(), None, self.weight, self.bias, self.eps, out)
        return out

    def add_norm(self, residual, delta, rows=None, write_back=True):
        if isinstance(delta, (Prenormed, Normed)):       # the stream holds the sum already
            delta = None
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=self.runtime.dtype, device=residual.device)
        kernels.add_layernorm(residual, delta, self.weight, self.bias, self.eps, out, rows, write_back)
        return out
