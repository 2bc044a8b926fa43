"""A short causal convolution on a mixer's input, added to it: the inner mixer reads ``h + conv(h)`` with

    conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j),   j = 0 .. taps - 1,   zeros before the sequence's start,

one filter of ``taps`` weights per channel, no bias. The last ``taps - 1`` rows of h are part of a sequence's
state: they lie first in the cache entry's per-sequence state, the inner mixer's own state after them (the inner
mixer gets a schedule entry whose ``state_offset`` says so). Everything is float32 arithmetic.

When the block's opening norm is elementwise (``dyt``), the block hands over the un-normed stream and norm and
convolution are one kernel; any other norm runs first and the convolution reads its result.
"""
from __future__ import annotations

import dataclasses
from typing import Dict

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, StateNeed, register_part


@register_part("mixer", "input_conv")
class InputConvolution(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, taps: int):
        super().__init__(build, spec)
        self.hidden, self.taps = int(hidden), int(taps)
        if not (1 <= self.taps <= build.kernels.DYT_MAX_TAPS):
            raise ValueError(f"the input convolution takes 1 to {build.kernels.DYT_MAX_TAPS} taps, got {taps}")
        self.inner = self.children["inner"]
        self.own_state = (self.taps - 1) * self.hidden
        self.p_conv = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"conv": ParamDecl((self.hidden, self.taps), role="vector", std=0.3)}

    def bind(self, t) -> None:
        self.p_conv = t["conv"].contiguous()

    def cache_need(self):
        return self.inner.cache_need()

    def state_need(self):
        inner = self.inner.state_need()
        total = self.own_state + (inner.numel if inner is not None else 0)
        return StateNeed(total) if total > 0 else None

    def planner(self):
        return self.inner.planner()

    def runs_beside(self, ctx) -> bool:
        return False

    def _inner_entry(self, entry):
        return dataclasses.replace(entry, state_offset=entry.state_offset + self.own_state)

    def _run_inner(self, y, ctx, entry, add):
        inner_entry = self._inner_entry(entry)
        if getattr(self.inner, "fuses_add", False):
            return self.inner.forward(y, ctx, inner_entry, add=add)
        out = self.inner.forward(y, ctx, inner_entry)
        if add is None:
            return out
        k = self.build.kernels
        return k.add_stream(add, out) if add.dtype != out.dtype else k.residual(add, out)

    def fuses_norm(self, norm) -> bool:
        return getattr(norm, "kind", None) == "dyt"

    def forward_stream(self, stream, norm, ctx, entry, add=None):
        """From the un-normed stream: the norm and the convolution in one kernel, then the inner mixer."""
        return self._run_inner(self._opened(stream, norm, ctx, entry), ctx, entry, add)

    def defers_sums(self) -> bool:
        return hasattr(self.inner, "forward_pending")

    def forward_stream_pending(self, stream, norm, ctx, entry, pending=None, pending_bias=None):
        """The same on a float32 stream whose last sum may not be formed yet (stream + (pending + pending_bias)), and
        without the sum at the end: (the stream as this block read it, the inner mixer's float32 result, its bias)."""
        if pending is not None:
            y, stream = self._opened(stream, norm, ctx, entry, pending, pending_bias)
        else:
            y = self._opened(stream, norm, ctx, entry)
        return (stream,) + tuple(self.inner.forward_pending(y, ctx, self._inner_entry(entry)))

    def _opened(self, stream, norm, ctx, entry, pending=None, pending_bias=None):
        k = self.build.kernels
        state = ctx.state_of(entry, self.own_state) if self.own_state else None
        return k.dyt(stream, norm.p_alpha, norm.p_weight, norm.p_bias, norm.out_dtype(stream), conv=self.p_conv, state=state,
                     slots=ctx.dev["slots"], batch=ctx.batch_c[0], single_tokens=ctx.is_decode, pending=pending,
                     pending_bias=pending_bias)

    def forward(self, x, ctx, entry, add=None):
        """From an input that is normed already."""
        raise NotImplementedError(
            "the input convolution runs under an elementwise opening norm (dyt), fused with it; a block with another "
            "norm needs a convolution kernel of its own, which this library does not have yet")
