"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` — the
reference's block (src/model/decoder_model.cpp:288-293).  The residual stream is
32-bit; every add is fused with the norm that follows it, so a block takes the
previous block's last delta as ``pending`` and hands its own on.
"""
from __future__ import annotations

from ..csrc import ops
from .base import Block, DeltaPair, FixedState, flatten_needs, count_needs, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    roles = ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm")

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        x = self.mixer_norm.add_forward(residual, pending)
        d = self.mixer.forward(x, batch, cache, writes_cache)
        x = self.feed_forward_norm.add_forward(residual, d)
        d = self.feed_forward.forward(x, batch)
        return residual, d


@register_block("stream_prenorm")
class StreamPreNormBlock(Block):
    """Pre-norm over one or several residual streams: each sublayer (the mixer, then the
    feed-forward if the layer has one) reads the streams through its connection, runs on the norm
    of what it read, and its result is written back through the same connection.  The connections
    stand in the roles ``mixer_connection`` and ``feed_forward_connection``; a layer without them
    has the ordinary residual sum.  The norms must take ``read=`` (``group_rmsnorm`` does).  A
    mixer whose last projection has a bias may leave it in ``output_bias`` instead of adding it:
    it then joins the stream write."""

    roles = ("mixer", "mixer_norm")

    def __init__(self, by_role, runtime):
        super().__init__(by_role, runtime)
        if self.feed_forward is not None and self.feed_forward_norm is None:
            raise ValueError("stream_prenorm: a feed-forward needs a feed_forward_norm")
        self.mixer_connection = self.by_role.get("mixer_connection")
        self.feed_forward_connection = self.by_role.get("feed_forward_connection")

    @staticmethod
    def _write(connection, delta, bias=None):
        from .connections import StreamWrite
        return connection.write(delta, bias) if connection is not None else StreamWrite(delta, bias)

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        c = self.mixer_connection
        x = self.mixer_norm.add_forward(residual, pending, read=c.w_in if c is not None else None)
        d = self.mixer.forward(x, batch, cache, writes_cache)
        pending = self._write(c, d, getattr(self.mixer, "output_bias", None))
        if self.feed_forward is not None:
            c = self.feed_forward_connection
            x = self.feed_forward_norm.add_forward(residual, pending, read=c.w_in if c is not None else None)
            pending = self._write(c, self.feed_forward.forward(x, batch))
        return residual, pending


@register_block("parallel")
class ParallelBlock(Block):
    """Mixer and feed-forward side by side on the same residual, each behind a norm of its own:
    ``h += mixer(norm1(h)) + feed_forward(norm2(h))``.  The two deltas travel on as one
    ``DeltaPair``; the next layer's pair of norms (or the final norm) adds both in 32-bit in the
    kernel that normalises.  A layer without a feed-forward has the mixer's branch only.  The
    norms must be ``rmsnorm`` parts (``pair_forward``)."""

    roles = ("mixer", "mixer_norm")

    def __init__(self, by_role, runtime):
        super().__init__(by_role, runtime)
        if self.feed_forward is not None and self.feed_forward_norm is None:
            raise ValueError("parallel: a feed-forward needs a feed_forward_norm")

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        x1, x2 = self.mixer_norm.pair_forward(residual, pending,
                                              self.feed_forward_norm if self.feed_forward is not None else None)
        d1 = self.mixer.forward(x1, batch, cache, writes_cache)
        d2 = self.feed_forward.forward(x2, batch) if self.feed_forward is not None else None
        return residual, DeltaPair(d1, d2)


@register_block("parallel_shared_norm")
class ParallelSharedNormBlock(Block):
    """Mixer and feed-forward side by side behind ONE norm: ``n = norm(h); h += mixer(n) + feed_forward(n)``.
    Both branches read the same normalised rows.  The two deltas travel on as one ``DeltaPair`` that the
    next layer's norm (or the final norm) adds in 32-bit in the kernel that normalises.  A layer without
    a feed-forward has the mixer's branch only."""

    roles = ("mixer", "mixer_norm")

    def __init__(self, by_role, runtime):
        super().__init__(by_role, runtime)
        if self.feed_forward_norm is not None:
            raise ValueError("parallel_shared_norm: the feed-forward reads the mixer's norm and has none of its own")

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        x = self.mixer_norm.add_forward(residual, pending)
        d1 = self.mixer.forward(x, batch, cache, writes_cache)
        d2 = self.feed_forward.forward(x, batch) if self.feed_forward is not None else None
        return residual, DeltaPair(d1, d2)


@register_block("postnorm_conv")
class PostNormConvBlock(Block):
    """The norms sit on the sublayers' OUTPUTS and the sublayers read the stream itself through a short
    convolution: ``x += norm1(mixer(c1(x)))``, then (if the layer has a feed-forward)
    ``x += norm2(feed_forward(c2(x)))``, with ``c(x) = x + conv(x)`` (the ``conv_read`` connections in the
    roles ``mixer_connection`` and ``feed_forward_connection``; a layer without one reads the stream's
    rounding).  The norms must have ``post_add`` (``rmsnorm`` has).  A mixer may hand back a
    ``ScaledPair`` (two branches side by side): the norm takes their weighted sum.

    The layer's state is its mixer's and, behind it, one ``FixedState`` with the convolutions' last rows
    (the mixer's connection first)."""

    roles = ("mixer", "mixer_norm")

    def __init__(self, by_role, runtime):
        super().__init__(by_role, runtime)
        if self.feed_forward is not None and self.feed_forward_norm is None:
            raise ValueError("postnorm_conv: a feed-forward needs a feed_forward_norm")
        self.mixer_connection = self.by_role.get("mixer_connection")
        self.feed_forward_connection = self.by_role.get("feed_forward_connection") if self.feed_forward is not None else None
        self.n_mixer_needs = count_needs(self.mixer.cache_need())
        self.conv_floats = sum(c.state_floats for c in (self.mixer_connection, self.feed_forward_connection)
                               if c is not None)

    def cache_need(self):
        own = FixedState((self.conv_floats,), tag="conv_read") if self.conv_floats else None
        needs = flatten_needs(self.mixer.cache_need(), own)
        return needs if len(needs) != 1 else needs[0]

    def _read(self, connection, residual, batch, conv_lane, offset, name):
        if connection is None:
            h = self.rt.buffer(name, tuple(residual.shape))
            h.copy_(residual)
            return h
        return connection.read(residual, batch, conv_lane.tensor if conv_lane is not None else residual, offset, name)

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        for d in ((pending.first, pending.second) if isinstance(pending, DeltaPair) else (pending,)):
            if d is not None:
                ops.residual_add(residual, d)
        lanes = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        n = self.n_mixer_needs
        mixer_cache = None if n == 0 else (lanes[0] if n == 1 else lanes[:n])
        conv_lane = lanes[n] if len(lanes) > n else None
        h = self._read(self.mixer_connection, residual, batch, conv_lane, 0, "block.read1")
        self.mixer_norm.post_add(residual, self.mixer.forward(h, batch, mixer_cache, writes_cache))
        if self.feed_forward is not None:
            off = self.mixer_connection.state_floats if self.mixer_connection is not None else 0
            h = self._read(self.feed_forward_connection, residual, batch, conv_lane, off, "block.read2")
            self.feed_forward_norm.post_add(residual, self.feed_forward.forward(h, batch))
        return residual, None
