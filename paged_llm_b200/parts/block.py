"""Pre-norm arrangement: x += mixer(norm_in(x)); x += ffn(norm_post(x))
(reference: pagedllm/model/llama.py:174-185).  Each residual sum is handed to
the following norm as a pending branch so that one kernel does both.  A layer
without a feed-forward (`feed_forward` None, no "post_mixer" norm) is
x += mixer(norm_in(x)) alone."""

from __future__ import annotations

from .base import Block, LazyNormed, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    NORM_NAMES = ("input", "post_mixer")

    def forward(self, x, pending, ctx, cache):
        h = self.norms["input"].add_forward(x, pending, ctx)
        if not self.mixer.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return x, a
        h = self.norms["post_mixer"].add_forward(x, a, ctx)
        if not self.feed_forward.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        f = self.feed_forward.forward(h, ctx)
        return x, f


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm in front of and behind each part: x += behind_mixer(mixer(input(x))), then
    x += behind_ffn(ffn(post_mixer(x))).  The norm behind a part travels with the branch (`LazyNormed`), so the
    norm that follows can do both norms and the sum in one kernel."""

    NORM_NAMES = ("input", "behind_mixer", "post_mixer", "behind_ffn")

    def forward(self, x, pending, ctx, cache):
        h = self.norms["input"].add_forward(x, pending, ctx)
        if not self.mixer.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        a = LazyNormed(self.mixer.forward(h, ctx, cache), self.norms["behind_mixer"])
        if self.feed_forward is None:
            return x, a
        h = self.norms["post_mixer"].add_forward(x, a, ctx)
        if not self.feed_forward.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        return x, LazyNormed(self.feed_forward.forward(h, ctx), self.norms["behind_ffn"])
