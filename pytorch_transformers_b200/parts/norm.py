"""Norm parts: LayerNorm and RMSNorm over the hidden axis, statistics in float32, and the Dynamic Tanh norm
(``dyt``: ``tanh(alpha x) * weight + bias`` with one learned scalar ``alpha``; elementwise, no statistics at all).

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

    def _stream(self, x) -> bool:
        """Is ``x`` a float32 residual stream of a model whose matrices are not float32? Its norm is then
        read in float32 and written in the model dtype."""
        import torch
        return x.dtype == torch.float32 and self.build.dtype != torch.float32

    def forward(self, x):
        if self._stream(x):
            return self.build.kernels.norm_stream(x, self.p_weight, self.p_bias, self.eps, self.kind, self.build.dtype)
        return self.build.kernels.norm(x, self.p_weight, self.p_bias, self.eps, self.kind)

    def forward_same(self, x):
        """The norm in ``x``'s own dtype: a float32 stream stays float32 (the norm of the embeddings, which is the
        stream's first value)."""
        return self.build.kernels.norm(x, self.p_weight, self.p_bias, self.eps, self.kind)

    def forward_sum(self, x, addend, other: "LayerNorm" = None):
        """Norm of ``x + addend``: returns (the sum, its norm[, ``other``'s norm of it]) from one kernel."""
        k = self.build.kernels
        if self._stream(x):
            total, y = k.norm_stream(x, self.p_weight, self.p_bias, self.eps, self.kind, self.build.dtype, addend=addend)
            return (total, y) if other is None else (total, y, other.forward(total))
        if other is not None and (other.kind != self.kind or other.eps != self.eps or other.size != self.size):
            total, y = k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, addend=addend)
            return total, y, other.forward(total)
        if other is not None:
            return k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, gain2=other.p_weight,
                          bias2=other.p_bias, addend=addend)
        return k.norm(x, self.p_weight, self.p_bias, self.eps, self.kind, addend=addend)

    def forward_pair(self, x, other: "LayerNorm"):
        """Two norms of the same input with the same statistics: one read, two outputs."""
        if other.kind != self.kind or other.eps != self.eps or other.size != self.size or self._stream(x):
            return self.forward(x), other.forward(x)
        return self.build.kernels.norm(x, self.p_weight, self.p_bias, self.eps, self.kind,
                                       gain2=other.p_weight, bias2=other.p_bias)


@register_part("norm", "rmsnorm")
class RMSNorm(LayerNorm):
    kind = "rmsnorm"

    def __init__(self, build: BuildContext, spec: PartSpec, size: int, eps: float, bias: bool = False,
                 one_plus: bool = False):
        super().__init__(build, spec, size, eps, bias)
        # the stored weight is the gain's distance from one: y = x / rms(x) * (1 + w). The device holds 1 + w (float32).
        self.one_plus = bool(one_plus)

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = super().param_decls()
        if self.one_plus:
            d["weight"] = ParamDecl((self.size,), role="vector", init="normal", std=0.1)
        return d

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.one_plus:
            self.p_weight = self.p_weight + 1.0


@register_part("norm", "dyt")
class DynamicTanh(Part):
    """y = tanh(alpha * x) * weight + bias, in float32; ``alpha`` is a scalar parameter. Nothing is reduced over the
    row, so a kernel that reads the rows anyway can form it on the way (``parts/input_conv.py`` does)."""
    kind = "dyt"
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, size: int, bias: bool = True):
        super().__init__(build, spec)
        self.size, self.has_bias = int(size), bool(bias)
        self.p_weight = self.p_bias = self.p_alpha = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"weight": ParamDecl((self.size,), role="vector", init="one_plus_normal", std=0.1),
             "alpha": ParamDecl((), role="vector", init="one_plus_normal", std=0.1)}
        if self.has_bias:
            d["bias"] = ParamDecl((self.size,), role="vector", init="normal", std=0.1)
        return d

    def out_dtype(self, x):
        """A float32 stream of a bfloat16 model is normed into bfloat16; anything else keeps its type."""
        import torch
        return self.build.dtype if x.dtype == torch.float32 else x.dtype

    def forward(self, x):
        return self.build.kernels.dyt(x, self.p_alpha, self.p_weight, self.p_bias, self.out_dtype(x))

    def forward_pending(self, base, pending, pending_bias=None):
        """The norm of base + (pending + pending_bias), float32 rows that have not been summed yet: (normed, sum), both
        out of one kernel."""
        return self.build.kernels.dyt(base, self.p_alpha, self.p_weight, self.p_bias, self.out_dtype(base), pending=pending,
                                      pending_bias=pending_bias)
