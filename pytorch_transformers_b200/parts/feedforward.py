"""Feed-forward parts. ``dense``: down(act(up(x))), no gating
(FalconMLP, src/transformers/models/falcon/modeling_falcon.py:565-578; activations by name,
src/transformers/activations.py:200-228)."""
from __future__ import annotations

from typing import Dict

from .base import BuildContext, ParamDecl, Part, PartSpec, register_part
from .linear import linear


@register_part("feed_forward", "dense")
class DenseFeedForward(Part):
    graph_safe = True
    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, inner: int, activation: str = "gelu",
                 bias: bool = False):
        super().__init__(build, spec)
        if activation not in build.kernels.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not supported "
                             f"(supported: {', '.join(build.kernels.ACTIVATIONS)})")
        self.hidden, self.inner, self.activation, self.has_bias = int(hidden), int(inner), activation, bool(bias)
        self.p_up_weight = self.p_up_bias = self.p_down_weight = self.p_down_bias = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"up.weight": ParamDecl((self.inner, self.hidden)), "down.weight": ParamDecl((self.hidden, self.inner))}
        if self.has_bias:
            d["up.bias"] = ParamDecl((self.inner,), role="vector")
            d["down.bias"] = ParamDecl((self.hidden,), role="vector")
        return d

    fuses_add = True

    def forward(self, x, ctx, add=None):
        k = self.build.kernels
        u = linear(k, x, self.p_up_weight, self.p_up_bias, self.activation)
        if callable(add):
            add = add()   # resolved as late as possible: the caller may still be producing it on another stream
        return linear(k, u, self.p_down_weight, self.p_down_bias, add=add)
