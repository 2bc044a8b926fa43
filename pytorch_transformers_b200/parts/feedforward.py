"""Feed-forward parts. ``dense``: down(act(up(x))), no gating
(FalconMLP, src/transformers/models/falcon/modeling_falcon.py:565-578; activations by name,
src/transformers/activations.py:200-228). ``gated``: down(act(gate(x)) * up(x)) with the activation by name.
``clamped_glu``: a gated unit with clamped branches."""
from __future__ import annotations

from typing import Dict

from .base import BuildContext, ParamDecl, Part, PartSpec, register_part
from .linear import linear, linear_pending


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

    def forward_pending(self, x, ctx):
        """The result as the last product's float32 sums and its bias, for a kernel that adds them to the stream later."""
        k = self.build.kernels
        u = linear(k, x, self.p_up_weight, self.p_up_bias, self.activation)
        return linear_pending(k, u, self.p_down_weight, self.p_down_bias)


@register_part("feed_forward", "clamped_glu")
class ClampedGatedFeedForward(Part):
    """A gated feed-forward with clamped branches:

        g = min(W_gate x, limit),  u = clamp(W_up x, -limit, limit),  y = W_down (g * sigmoid(alpha g) * (u + 1)).

    Gate and up are one matrix and one product; the unit between the products is one kernel. ``forward``
    returns the last product's float32 sums unrounded when asked (``wide_out``), for a norm that follows."""
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, inner: int, limit: float, alpha: float = 1.702,
                 wide_out: bool = False):
        super().__init__(build, spec)
        self.hidden, self.inner, self.limit, self.alpha = int(hidden), int(inner), float(limit), float(alpha)
        self.wide_out = bool(wide_out)
        if not self.limit > 0:
            raise ValueError(f"the clamp's limit must be positive, got {limit}")
        self.p_gate_up = self.p_down = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"gate": ParamDecl((self.inner, self.hidden)), "up": ParamDecl((self.inner, self.hidden)),
                "down": ParamDecl((self.hidden, self.inner))}

    def bind(self, t) -> None:
        import torch
        self.p_gate_up = torch.cat([t["gate"], t["up"]]).contiguous()
        self.p_down = t["down"]

    def forward(self, x, ctx):
        k = self.build.kernels
        y = k.glu_clamp(linear(k, x, self.p_gate_up), self.limit, self.alpha)
        return linear(k, y, self.p_down, wide_out=self.wide_out)


@register_part("feed_forward", "gated")
class GatedFeedForward(Part):
    """y = W_down (act(W_gate x) * (W_up x)), ``activation`` by name (the tanh form of GELU, silu, ...). Gate and up are
    one matrix and one product; the unit between the products is one kernel. With ``wide_out`` the last product's
    float32 sums are returned unrounded (for a float32 stream, or for a kernel that weighs and adds them)."""
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, inner: int, activation: str = "silu",
                 wide_out: bool = False):
        super().__init__(build, spec)
        if activation not in build.kernels.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not supported "
                             f"(supported: {', '.join(build.kernels.ACTIVATIONS)})")
        self.hidden, self.inner, self.activation, self.wide_out = int(hidden), int(inner), activation, bool(wide_out)
        self.p_gate_up = self.p_down = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"gate": ParamDecl((self.inner, self.hidden)), "up": ParamDecl((self.inner, self.hidden)),
                "down": ParamDecl((self.hidden, self.inner))}

    def bind(self, t) -> None:
        import torch
        self.p_gate_up = torch.cat([t["gate"], t["up"]]).contiguous()
        self.p_down = t["down"]

    def forward(self, x, ctx, add=None):
        k = self.build.kernels
        y = k.glu_act(linear(k, x, self.p_gate_up), self.activation)
        if callable(add):
            add = add()
        if add is not None:
            return linear(k, y, self.p_down, add=add)
        return linear(k, y, self.p_down, wide_out=self.wide_out)

    def forward_pending(self, x, ctx):
        """The result as the last product's float32 sums (and no bias), for a kernel that adds them to the stream later."""
        k = self.build.kernels
        return linear_pending(k, k.glu_act(linear(k, x, self.p_gate_up), self.activation), self.p_down)
