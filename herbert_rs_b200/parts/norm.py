"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, in float
(crates/backends/backend_common/src/kernels.rs:54-64), and the layer norm with a weight and no bias."""

from __future__ import annotations

from .. import ops
from ..registry import register_part
from .base import Norm, ParamSpec


class RMSNorm(Norm):
    def __init__(self, spec, rt):
        self.dim, self.eps, self.rt = spec.dim, spec.eps, rt
        self.name = getattr(spec, "weight_name", "weight")
        self.weight = None

    def param_specs(self):
        return {self.name: ParamSpec((self.dim,), role="vector", init="ones_noise")}

    def load(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def weight_bytes(self):
        return self.dim * 4

    def forward(self, x, out, rows=None):
        ops.rmsnorm(x, self.weight, out, self.eps, rows)

    def shareable(self):
        return (self.weight, self.eps)


class LayerNorm(RMSNorm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w, no bias, in float (var: mean of squared deviations)."""

    def forward(self, x, out, rows=None):
        ops.layernorm(x, self.weight, out, self.eps, rows)

    def shareable(self):
        return None         # the products' shared norm is the RMS form only


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
