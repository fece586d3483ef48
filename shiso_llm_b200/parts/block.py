"""Arrangements of norm, mixer, feed-forward and the residual stream in one layer.

``pre_norm``: ``h = x + mixer(norm(x))``, ``x' = h + ff(norm(h))`` with no
post-norms (crates/shiso-models/src/lfm2/config.rs:184; the layer loop at
crates/shiso-engine/src/layers.rs:2003-2294).  A block only marks its outputs as
pending on the stream; the next norm adds them while it normalises.

``output_norm``: the norm stands behind each sublayer, not before it: ``h = x + norm1(mixer(x))``,
``x' = h + norm2(ff(h))``; the sublayers read the stream itself.  One kernel per sublayer takes
the norm of the output, adds it to the float32 residual and writes the new residual out in the
compute type for the next reader.
"""

from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, env, layer):
        super().__init__(spec, env)
        self.name = layer.name
        self.mixer_norm = NORMS.build(layer.mixer_norm, env)
        self.mixer = MIXERS.build(layer.mixer, env)
        self.feed_forward = None
        self.ff_norm = None
        if layer.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, env)
            self.ff_norm = NORMS.build(layer.feed_forward_norm, env)

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        specs = []
        for part in self.sub_parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors):
        for part in self.sub_parts():
            part.bind(tensors)

    def mixer_part(self):
        return self.mixer

    def forward(self, stream, step, cache):
        x = stream.normed(self.mixer_norm, getattr(self.mixer, "takes_deferred_norm", False))
        stream.add(self.mixer.forward(x, step, cache))
        if self.feed_forward is not None:
            x = stream.normed(self.ff_norm, getattr(self.feed_forward, "takes_deferred_norm", False))
            stream.add(self.feed_forward.forward(x, step))


@BLOCKS.register("parallel_pre_norm")
class ParallelPreNormBlock(Block):
    """``x' = x + mixer(h) + ff(h)`` with ``h = norm(x)``: one norm, read by both sublayers.
    Both outputs wait on the stream together; the next norm adds them in float32 while it
    normalises.  A layer without a feed-forward leaves the mixer's output alone."""

    def __init__(self, spec, env, layer):
        super().__init__(spec, env)
        self.name = layer.name
        if layer.feed_forward_norm is not None:
            raise ValueError(f"layer {layer.name}: a parallel layer has one norm, read by the mixer and the feed-forward")
        self.norm = NORMS.build(layer.mixer_norm, env)
        self.mixer = MIXERS.build(layer.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, env) if layer.feed_forward is not None else None

    def sub_parts(self):
        return [p for p in (self.norm, self.mixer, self.feed_forward) if p is not None]

    def tensor_specs(self):
        specs = []
        for part in self.sub_parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors):
        for part in self.sub_parts():
            part.bind(tensors)

    def mixer_part(self):
        return self.mixer

    def forward(self, stream, step, cache):
        h = stream.normed(self.norm)
        mixed = self.mixer.forward(h, step, cache)
        if self.feed_forward is None:
            stream.add(mixed)
        else:
            stream.add((mixed, self.feed_forward.forward(h, step)))


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """``x <- x + norm(sublayer(x))`` for the mixer and then for the feed-forward (if any)."""

    def __init__(self, spec, env, layer):
        super().__init__(spec, env)
        self.name = layer.name
        self.mixer_norm = NORMS.build(layer.mixer_norm, env)
        self.mixer = MIXERS.build(layer.mixer, env)
        self.feed_forward = self.ff_norm = None
        if layer.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, env)
            self.ff_norm = NORMS.build(layer.feed_forward_norm, env)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"layer {layer.name}: {type(norm).__name__} cannot add the norm of an output to the stream")

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        specs = []
        for part in self.sub_parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors):
        for part in self.sub_parts():
            part.bind(tensors)

    def mixer_part(self):
        return self.mixer

    @staticmethod
    def _rows(y):
        return y.materialize() if hasattr(y, "materialize") else y

    def forward(self, stream, step, cache):
        x = stream.rows(self.env)
        y = self._rows(self.mixer.forward(x, step, cache))
        stream.current = self.mixer_norm.add_normed(stream.residual, y)
        if self.feed_forward is not None:
            y = self._rows(self.feed_forward.forward(stream.rows(self.env), step))
            stream.current = self.ff_norm.add_normed(stream.residual, y)
        if stream.observer is not None:
            stream.observer(stream)
