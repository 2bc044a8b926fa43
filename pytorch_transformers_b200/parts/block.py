"""Block parts: how norms, mixer and feed-forward are arranged around the residual stream.

``parallel``: mixer and feed-forward both read normed copies of the block input, and the
output is ``(x + mixer) + ff``, each sum formed in float32 in the epilogue of the kernel that
produces the second term; the reference adds in the order ``x + (ff + mixer)`` (FalconDecoderLayer with parallel attention,
src/transformers/models/falcon/modeling_falcon.py:630-634, 652-654, 673-676); with a
``norm_ff`` child the feed-forward has its own norm of x, else it shares the mixer's; without a ``feed_forward`` child
the block is ``x + mixer``.
``sequential``: ``r = x + mixer(norm(x))``, then ``r + ff(norm_ff(r))`` (:656-659, 676); without a
``feed_forward`` child the block ends at ``r``.
Sums are formed in float32 and rounded once; where the model keeps its residual stream in float32
(``ModelSpec.stream_float32``) they are not rounded at all.
"""
from __future__ import annotations

from .base import BuildContext, DeferredSum, NormedStream, Part, PartSpec, register_part, resolve


def _plus(kernels, part, base, *args):
    """part.forward(*args) + base. A part that sets ``fuses_add`` sums ``base`` into its own last
    kernel's float32 epilogue; for any other part the sum is a kernel of its own."""
    if getattr(part, "fuses_add", False):
        return part.forward(*args, add=base)
    y = part.forward(*args)
    if base.dtype != y.dtype:       # a float32 stream takes a branch's result of the model dtype
        return kernels.add_stream(base, y)
    return kernels.residual(base, y)


@register_part("block", "parallel")
class ParallelBlock(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec):
        super().__init__(build, spec)
        self.norm_mixer = self.children["norm_mixer"]
        self.norm_ff = self.children.get("norm_ff")
        self.mixer = self.children["mixer"]
        self.feed_forward = self.children.get("feed_forward")     # a block without one is x + mixer(norm(x))

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        side = getattr(ctx, "side_stream", None)
        two_streams = (side is not None and self.feed_forward is not None and getattr(self.mixer, "fuses_add", False)
                       and getattr(self.feed_forward, "fuses_add", False) and hasattr(self.norm_mixer, "forward_sum"))
        can_join = hasattr(self.norm_mixer, "forward_sum")
        if isinstance(x, DeferredSum) and can_join:
            # join the previous block's two terms and norm the sum in one kernel
            x.join(x.base.device)
            outs = self.norm_mixer.forward_sum(x.base, x.pending, self.norm_ff)
            ctx.keep_alive.append((x.base, x.pending))
            x, a = outs[0], outs[1]
            m = outs[2] if self.norm_ff is not None else a
        else:
            x = resolve(k, x)
            if self.norm_ff is not None:
                a, m = self.norm_mixer.forward_pair(x, self.norm_ff)
            else:
                a = self.norm_mixer.forward(x)
                m = a
        if two_streams:
            return self._forward_two_streams(x, a, m, ctx, entry, side)
        mixed = _plus(k, self.mixer, x, a, ctx, entry)           # x + mixer
        if self.feed_forward is None:
            return mixed
        # (x + mixer) + feed-forward: the last sum is left to whoever needs the value (the next
        # block's norm adds and norms in one kernel; the model's end adds)
        return DeferredSum(mixed, self.feed_forward.forward(m, ctx))

    def _forward_two_streams(self, x, a, m, ctx, entry, side):
        """Steps of a few tokens are bound by the read of the weights, and the mixer's chain of small
        kernels (projection, cache write, attention) leaves the memory system idle. Mixer and
        feed-forward are independent, so the mixer runs on a second stream while the feed-forward
        streams its weights on the first; the feed-forward takes ``x`` into its last epilogue and
        the mixer's result stays pending: the block returns ``DeferredSum(x + ff, mixer)``, which
        the next block's norm (or the model's end) joins. In a captured graph these are two
        parallel branches per block. The mixer's launches come first: with the feed-forward's first,
        its blocks take the SMs and the mixer's short kernels queue behind them (15 % slower).
        Tensors that cross streams stay referenced until the step ends."""
        import torch
        main = torch.cuda.current_stream(x.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            mixed = self.mixer.forward(a, ctx, entry)
        t = self.feed_forward.forward(m, ctx, add=x)
        ctx.keep_alive.append((a, m, x, mixed, t))
        return DeferredSum(t, mixed, side)


@register_part("block", "sequential")
class SequentialBlock(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec):
        super().__init__(build, spec)
        self.norm_mixer = self.children["norm_mixer"]
        self.mixer = self.children["mixer"]
        # a block without a feed-forward is its mixer's half alone
        self.feed_forward = self.children.get("feed_forward")
        self.norm_ff = self.children["norm_ff"] if self.feed_forward is not None else None

    def _defers(self, x) -> bool:
        """Elementwise norms on a float32 stream, under a mixer and a feed-forward that can leave their last sum to the
        next norm's kernel: no sum of this block is a kernel of its own."""
        import torch
        fuses = getattr(self.mixer, "fuses_norm", None)
        base = x.base if isinstance(x, DeferredSum) else x
        return (fuses is not None and fuses(self.norm_mixer) and getattr(self.mixer, "defers_sums", lambda: False)()
                and torch.is_tensor(base) and base.dtype == torch.float32
                and (self.feed_forward is None or (hasattr(self.norm_ff, "forward_pending")
                                                   and hasattr(self.feed_forward, "forward_pending"))))

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        if self._defers(x):
            # stream + (what the block before left) is formed by the opening norm's kernel, stream + mixer by the
            # feed-forward's norm, and stream + feed-forward is left to the next block (or the model's end)
            pending = bias = None
            if isinstance(x, DeferredSum) and x.pending.dtype == x.base.dtype:
                x.join(x.base.device)
                x, pending, bias = x.base, x.pending, x.bias
            else:
                x = resolve(k, x)
            x, mixed, mixed_bias = self.mixer.forward_stream_pending(x, self.norm_mixer, ctx, entry, pending, bias)
            if self.feed_forward is None:
                return DeferredSum(x, mixed, bias=mixed_bias)
            normed, r = self.norm_ff.forward_pending(x, mixed, mixed_bias)
            out, out_bias = self.feed_forward.forward_pending(normed, ctx)
            return DeferredSum(r, out, bias=out_bias)
        x = resolve(k, x)
        fuses = getattr(self.mixer, "fuses_norm", None)
        if fuses is not None and fuses(self.norm_mixer):
            # the mixer forms the opening norm in its own first kernel (an elementwise norm under a short convolution)
            r = self.mixer.forward_stream(x, self.norm_mixer, ctx, entry, add=x)
        else:
            r = _plus(k, self.mixer, x, self.norm_mixer.forward(x), ctx, entry)
        if self.feed_forward is None:
            return r
        return _plus(k, self.feed_forward, r, self.norm_ff.forward(r), ctx)


@register_part("block", "sandwich")
class SandwichBlock(Part):
    """A norm before and after each sublayer, and a fixed multiplier on what a sublayer adds:

        x <- x + mult * post_mixer(mixer(norm_mixer(x)));      x <- x + mult * post_ff(ff(norm_ff(x)))

    on a float32 residual stream (``ModelSpec.stream_float32``). All four norms are RMS norms. The closing norm of
    the mixer's result, the stream's sum and the feed-forward's opening norm are one kernel; so are the closing norm
    of the feed-forward's result and the sum, which also forms the opening norm of the next block when that is a
    sandwich block too (``NormedStream``). A block without ``feed_forward`` ends after its first half."""
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, mult: float = 1.0):
        super().__init__(build, spec)
        self.mult = float(mult)
        self.norm_mixer, self.post_mixer, self.mixer = (self.children[n] for n in ("norm_mixer", "post_mixer", "mixer"))
        self.feed_forward = self.children.get("feed_forward")
        self.norm_ff = self.children["norm_ff"] if self.feed_forward is not None else None
        self.post_ff = self.children["post_ff"] if self.feed_forward is not None else None
        for n in (self.norm_mixer, self.post_mixer, self.norm_ff, self.post_ff):
            if n is not None and (getattr(n, "kind", None) != "rmsnorm" or n.has_bias):
                raise ValueError("the sandwich block's norms are RMS norms without bias")

    def forward(self, x, ctx, entry):
        import torch
        k = self.build.kernels
        opened = x.normed if isinstance(x, NormedStream) and x.by is self.norm_mixer else None
        x = resolve(k, x)
        if x.dtype != torch.float32:
            raise ValueError("the sandwich block runs on a float32 residual stream")
        y = self.mixer.forward(opened if opened is not None else self.norm_mixer.forward(x), ctx, entry)
        if self.feed_forward is None:
            return self._close(ctx, x, y, self.post_mixer)
        x, h = k.post_norm_add(x, y, self.post_mixer.p_weight, self.post_mixer.eps, self.mult,
                               gain_next=self.norm_ff.p_weight, eps_next=self.norm_ff.eps, next_dtype=self.build.dtype)
        return self._close(ctx, x, self.feed_forward.forward(h, ctx), self.post_ff)

    def _close(self, ctx, x, y, post):
        """The block's last sum; with the next block's opening norm when that block is of this kind."""
        k = self.build.kernels
        nxt = getattr(ctx, "next_block", None)
        if isinstance(nxt, SandwichBlock):
            norm = nxt.norm_mixer
            x, h = k.post_norm_add(x, y, post.p_weight, post.eps, self.mult, gain_next=norm.p_weight, eps_next=norm.eps,
                                   next_dtype=self.build.dtype)
            return NormedStream(x, h, norm)
        return k.post_norm_add(x, y, post.p_weight, post.eps, self.mult)
