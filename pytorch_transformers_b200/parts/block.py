"""Block parts: how norms, mixer and feed-forward are arranged around the residual stream.

``parallel``: mixer and feed-forward both read normed copies of the block input, and the
output is ``(x + mixer) + ff``, each sum formed in float32 in the epilogue of the kernel that
produces the second term; the reference adds in the order ``x + (ff + mixer)`` (FalconDecoderLayer with parallel attention,
src/transformers/models/falcon/modeling_falcon.py:630-634, 652-654, 673-676); with a
``norm_ff`` child the feed-forward has its own norm of x, else it shares the mixer's.
``sequential``: ``r = x + mixer(norm(x))``, then ``r + ff(norm_ff(r))`` (:656-659, 676).
Sums are formed in float32 and rounded once.
"""
from __future__ import annotations

from .base import BuildContext, DeferredSum, Part, PartSpec, register_part, resolve


def _plus(kernels, part, base, *args):
    """part.forward(*args) + base. A part that sets ``fuses_add`` sums ``base`` into its own last
    kernel's float32 epilogue; for any other part the sum is a kernel of its own."""
    if getattr(part, "fuses_add", False):
        return part.forward(*args, add=base)
    return kernels.residual(base, part.forward(*args))


@register_part("block", "parallel")
class ParallelBlock(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec):
        super().__init__(build, spec)
        self.norm_mixer = self.children["norm_mixer"]
        self.norm_ff = self.children.get("norm_ff")
        self.mixer = self.children["mixer"]
        self.feed_forward = self.children["feed_forward"]

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        side = getattr(ctx, "side_stream", None)
        two_streams = (side is not None and getattr(self.mixer, "fuses_add", False)
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
        self.norm_ff = self.children["norm_ff"]
        self.mixer = self.children["mixer"]
        self.feed_forward = self.children["feed_forward"]

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        x = resolve(k, x)
        r = _plus(k, self.mixer, x, self.norm_mixer.forward(x), ctx, entry)
        return _plus(k, self.feed_forward, r, self.norm_ff.forward(r), ctx)
