"""Pre-norm residual arrangement of one layer.

``h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))`` (src/cloud_engine/model.py:212-220).
The residual stream is float32 and each add is fused into the norm that follows it, so
a layer leaves its last update pending for whoever normalises next.
"""

from __future__ import annotations

from .base import Block, register_part


def _normalise(norm, consumer, residual, pending, ctx):
    """A consumer that declares ``takes_normed_input`` may get the norm un-computed (see
    ``Norm.forward_lazy``); every other pairing runs the norm's kernel."""
    lazy = getattr(norm, "forward_lazy", None)
    if lazy is not None and getattr(consumer, "takes_normed_input", False):
        return lazy(residual, pending, ctx)
    return norm.forward(residual, pending, ctx)


def _lazy_gain(norm, consumer):
    """The gain a projection may pre-multiply with for ``norm``, if ``consumer`` can finish it."""
    if getattr(consumer, "takes_normed_input", False) and hasattr(norm, "forward_lazy"):
        return getattr(norm, "lazy_gain", None)
    return None


class PreNormResidual(Block):
    """``feed_forward`` and ``feed_forward_norm`` may both be left out: the layer is then its mixer sublayer alone."""

    slots = ("mixer", "mixer_norm")
    kernels_through_ops = True   # the block itself launches nothing

    def __init__(self, parts, **params) -> None:
        super().__init__(parts, **params)
        if ("feed_forward" in parts) != ("feed_forward_norm" in parts):
            raise ValueError("PreNormResidual: a feed-forward and its norm come together or not at all")
        self.has_feed_forward = "feed_forward" in parts

    def entry_gain(self):
        return _lazy_gain(self.mixer_norm, self.mixer)

    def forward(self, residual, pending, ctx, binding):
        sink = getattr(ctx, "residual_sink", None)
        if sink is not None:
            # after a projection of this block comes a product of this engine (the feed-forward's, or
            # the next layer's first) or a norm kernel: before their dependency wait they ask for
            # weights only, so the projection may let them start early
            sink.early_trigger = True
        x = _normalise(self.mixer_norm, self.mixer, residual, pending, ctx)
        if not self.has_feed_forward:
            if sink is not None:   # the mixer's sum is read next by whoever comes after this layer
                sink.gain = sink.following_gain
            return self.mixer.forward(x, ctx, binding)
        if sink is not None:   # the mixer's sum is read next by this layer's second norm
            sink.gain = _lazy_gain(self.feed_forward_norm, self.feed_forward)
        update = self.mixer.forward(x, ctx, binding)
        x = _normalise(self.feed_forward_norm, self.feed_forward, residual, update, ctx)
        if sink is not None:   # the feed-forward's sum by whoever comes after this layer
            sink.gain = sink.following_gain
        return self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual, replace=True)


class StreamResidual(Block):
    """Pre-norm layer over one residual stream or several: ``mixer`` and ``mixer_norm`` always,
    ``feed_forward`` with ``feed_forward_norm`` if the layer has one, and per sublayer a
    ``*_connection`` if the streams are read and written through hyper-connections (without one a
    sublayer reads the sum of the streams and its result is added to each, which with one stream is
    ``x + sublayer(norm(x))``).  Every write to the streams is left pending for the norm that reads
    them next; the norms are ``StreamRMSNorm`` (they take ``read`` weights)."""

    slots = ("mixer", "mixer_norm")

    def forward(self, residual, pending, ctx, binding):
        from ..lazy import StreamUpdate

        for name in ("mixer", "feed_forward"):
            part = self.parts.get(name)
            if part is None:
                continue
            connection = self.parts.get(name + "_connection")
            read = connection.read_weights() if connection is not None else None
            x = self.parts[name + "_norm"].forward(residual, pending, ctx, read=read)
            y = part.forward(x, ctx, binding) if name == "mixer" else part.forward(x, ctx)
            pending = connection.pending(y) if connection is not None else StreamUpdate(y)
        return pending


register_part("block", "stream_residual", StreamResidual, replace=True)


class ParallelResidual(Block):
    """One norm, and both sublayers read its output: ``x <- x + (mixer(h) + feed_forward(h))`` with
    ``h = norm(x)``; a layer without a feed-forward is ``x <- x + mixer(h)``.  Both results are float32
    and stay apart: they travel to the next norm as a ``Partials`` of two terms, whose kernel adds
    them up and into the stream in float32."""

    slots = ("mixer", "mixer_norm")

    def forward(self, residual, pending, ctx, binding):
        from ..lazy import Partials

        sink = getattr(ctx, "residual_sink", None)
        if sink is not None:
            ctx.residual_sink = None      # nothing of this block adds itself into the stream
        x = self.mixer_norm.forward(residual, pending, ctx)
        mixed = self.mixer.forward(x, ctx, binding)
        feed_forward = self.parts.get("feed_forward")
        if feed_forward is None:
            result = Partials(mixed, 1, mixed.shape[0], mixed.shape[1], None)
        else:
            result = Partials.of_terms(mixed, feed_forward.forward(x, ctx))
        ctx.residual_sink = sink
        return result


register_part("block", "parallel_residual", ParallelResidual, replace=True)
