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

from .base import BuildContext, Part, PartSpec, register_part


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
        if self.norm_ff is not None:
            a, m = self.norm_mixer.forward_pair(x, self.norm_ff)
        else:
            a = self.norm_mixer.forward(x)
            m = a
        k = self.build.kernels
        mixed = _plus(k, self.mixer, x, a, ctx, entry)           # x + mixer
        return _plus(k, self.feed_forward, mixed, m, ctx)        # (x + mixer) + feed-forward


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
        r = _plus(k, self.mixer, x, self.norm_mixer.forward(x), ctx, entry)
        return _plus(k, self.feed_forward, r, self.norm_ff.forward(r), ctx)
