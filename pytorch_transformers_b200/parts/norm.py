"""Norm parts: LayerNorm and RMSNorm over the hidden axis, statistics in float32.

``torch.nn.LayerNorm(hidden, eps)`` is every norm of the reference's Falcon
(src/transformers/models/falcon/modeling_falcon.py:603-612, 843): biased variance, gain and bias.
"""
from __future__ import annotations

from typing import Dict

from .base import BuildContext, ParamDecl, Part, PartSpec, register_part


@register_part("norm", "layernorm")
class LayerNorm(Part):
    kind = "layernorm"
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, size: int, eps: float, bias: bool = True):
        super().__init__(build, spec)
        self.size, self.eps, self.has_bias = int(size), float(eps), bool(bias)
        self.p_weight = None
        self.p_bias = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"weight": ParamDecl((self.size,), role="vector", init="one_plus_normal")}
        if self.has_bias:
            d["bias"] = ParamDecl((self.size,), role="vector", init="normal")
        return d

    def forward(self, x):
        return self.build.kernels.norm(x, self.p_weight, self.p_bias, self.eps, self.kind)

    def forward_sum(self, x, addend, other: "LayerNorm" = None):
        """Norm of ``x + addend``: returns (the sum, its norm[, ``other``'s norm of it]) from one kernel."""
        k = self.build.kernels
        if other is not None and (other.kind != self.kind or other.eps != self.eps or other.size != self.size):
            total, y = k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, addend=addend)
            return total, y, other.forward(total)
        if other is not None:
            return k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, gain2=other.p_weight,
                          bias2=other.p_bias, addend=addend)
        return k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, addend=addend)

    def forward_pair(self, x, other: "LayerNorm"):
        """Two norms of the same input with the same statistics: one read, two outputs."""
        if other.kind != self.kind or other.eps != self.eps or other.size != self.size:
            return self.forward(x), other.forward(x)
        return self.build.kernels.norm(x, self.p_weight, self.p_bias, self.eps, self.kind,
                                       gain2=other.p_weight, bias2=other.p_bias)


@register_part("norm", "rmsnorm")
class RMSNorm(LayerNorm):
    kind = "rmsnorm"

    def __init__(self, build: BuildContext, spec: PartSpec, size: int, eps: float, bias: bool = False):
        super().__init__(build, spec, size, eps, bias)
