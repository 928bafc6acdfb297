"""Arrangements of a layer's parts. The reference's only one (engine/model.py:340-349):
norm, mixer, add; norm, feed-forward, add. The residual sum is made in 32-bit inside the
epilogue of each branch's last product."""

from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("pre_norm_residual")
class PreNormResidual(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, hidden, layer, cache):
        # `hidden` may be a product that is still to be summed; the norm's kernel sums it, and
        # `materialized` then hands out the summed tensor without another launch.
        normed = layer.mixer_norm.forward(ctx, hidden)
        hidden = layer.mixer.forward(ctx, normed, ctx.ops.materialized(hidden), cache)
        normed = layer.feed_forward_norm.forward(ctx, hidden)
        return layer.feed_forward.forward(ctx, normed, ctx.ops.materialized(hidden))


@BLOCKS.register("parallel_residual")
class ParallelResidual(Block):
    """One norm whose output both branches read: x <- x + mixer(norm(x)) + ff(norm(x)). Each
    branch's last product adds what came before it in its epilogue, in the residual's dtype
    (float32 when the embedding makes a float32 stream)."""

    roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, ctx, hidden, layer, cache):
        hidden = ctx.ops.materialized(hidden)
        normed = layer.norm.forward(ctx, hidden)
        hidden = layer.mixer.forward(ctx, normed, hidden, cache)
        return layer.feed_forward.forward(ctx, normed, ctx.ops.materialized(hidden))


@BLOCKS.register("mixer_residual")
class MixerResidual(Block):
    """A layer without a feed-forward: x <- x + mixer(norm(x))."""

    roles = {"norm": "norm", "mixer": "mixer"}

    def forward(self, ctx, hidden, layer, cache):
        # the norm may sum a product that is still in its splits; `materialized` then hands out that sum
        normed = layer.norm.forward(ctx, hidden)
        return layer.mixer.forward(ctx, normed, ctx.ops.materialized(hidden), cache)


@BLOCKS.register("hyper_connected")
class HyperConnected(Block):
    """Several residual streams instead of one. Each sublayer reads a weighted sum of the streams
    through its norm (a `stream_rms_norm`), and its `connection` part writes the output back: every
    new stream is a mix of the old ones plus a multiple of the output. The sublayers get no residual
    and leave their output in float32; the write stays pending until the next read, which does
    both in one kernel."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_merge": "connection",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_merge": "connection"}

    def forward(self, ctx, hidden, layer, cache):
        out = layer.mixer.forward(ctx, layer.mixer_norm.forward(ctx, hidden), None, cache)
        hidden = layer.mixer_merge.forward(ctx, ctx.ops.materialized(hidden), out)
        out = layer.feed_forward.forward(ctx, layer.feed_forward_norm.forward(ctx, hidden), None)
        return layer.feed_forward_merge.forward(ctx, ctx.ops.materialized(hidden), out)


@BLOCKS.register("hyper_connected_mixer")
class HyperConnectedMixer(Block):
    """A hyper-connected layer without a feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_merge": "connection"}

    def forward(self, ctx, hidden, layer, cache):
        out = layer.mixer.forward(ctx, layer.mixer_norm.forward(ctx, hidden), None, cache)
        return layer.mixer_merge.forward(ctx, ctx.ops.materialized(hidden), out)


@BLOCKS.register("sandwich_residual")
class SandwichResidual(Block):
    """A norm on both sides of each sublayer: x <- x + m * norm_b(mixer(norm_a(x))), then the same
    around the feed-forward, with the layer's `residual_mult` m (`params` of the LayerSpec; 1 when
    absent). The sublayers get no residual and leave float32; the norm after a sublayer adds its
    result to the stream (`add_to`, or for a norm without one its `forward` and a plain scaled sum),
    and that sum stays pending until the next norm reads the stream."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_out_norm": "norm"}

    def _add(self, ctx, norm, stream, y):
        mult = float(self.params.get("residual_mult", 1.0))
        if hasattr(norm, "add_to"):
            return norm.add_to(ctx, stream, y, mult)
        return ctx.ops.residual_add(stream, norm.forward(ctx, ctx.ops.materialized(y)), mult)

    def forward(self, ctx, hidden, layer, cache):
        normed = layer.mixer_norm.forward(ctx, hidden)
        out = layer.mixer.forward(ctx, normed, None, cache)
        hidden = self._add(ctx, layer.mixer_out_norm, ctx.ops.materialized(hidden), out)
        normed = layer.feed_forward_norm.forward(ctx, hidden)
        out = layer.feed_forward.forward(ctx, normed, None)
        return self._add(ctx, layer.feed_forward_out_norm, ctx.ops.materialized(hidden), out)


@BLOCKS.register("sandwich_residual_mixer")
class SandwichResidualMixer(SandwichResidual):
    """A sandwich-normed layer without a feed-forward."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm"}

    def forward(self, ctx, hidden, layer, cache):
        normed = layer.mixer_norm.forward(ctx, hidden)
        out = layer.mixer.forward(ctx, normed, None, cache)
        return self._add(ctx, layer.mixer_out_norm, ctx.ops.materialized(hidden), out)
