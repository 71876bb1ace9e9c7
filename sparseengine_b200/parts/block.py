"""Arrangement of a layer's parts in a block.

``pre_norm``: the model carries ``(hidden, residual)``; the first block takes
``residual = hidden``; afterwards each norm call adds the last sublayer's output to the
residual (32-bit add, rounded to the activation dtype) and normalises the unrounded sum
(src/sparseengine/models/minimax_m2.py:381-397).  Another arrangement registers under
another name in ``ARRANGEMENTS``: a class built from ``(LayerSpec, dtype)`` with ``parts()``
(name -> part: the model lists parameters and cache needs from it; the part named ``mixer`` is
the one that may ask for pages or state), ``forward(hidden, residual, step, slot)`` ->
``(hidden, residual)``, and an attribute ``mixer``.  Parts beyond the four of ``pre_norm`` come
from ``LayerSpec.extra``.

``post_norm`` (:class:`PostNormBlock`), ``pre_norm_stream`` (:class:`PreNormStreamBlock`) and
``sublayer_norm`` (:class:`SublayerNormBlock`) are the arrangements over a 32-bit stream,
``stream_mix`` (:class:`StreamMixBlock`) the one over several such streams.
"""
from __future__ import annotations

import torch

from .base import make_feed_forward, make_mixer, make_norm


class PreNormBlock:
    def __init__(self, spec, dtype):
        self.spec = spec
        self.mixer = make_mixer(spec.mixer, dtype)
        self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)

    def parts(self) -> dict:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, hidden, residual, step, slot):
        x, residual = self.mixer_norm.forward(hidden, residual)
        hidden = self.mixer.forward(x, step, slot)
        x, residual = self.feed_forward_norm.forward(hidden, residual)
        hidden = self.feed_forward.forward(x, step)
        return hidden, residual


class PostNormBlock:
    """Norm after the sum, over a 32-bit stream: ``x <- norm(a * x + mixer(x))``, then (if the layer
    has a feed-forward) ``x <- norm(a * x + feed_forward(x))`` with ``a = residual_scale``; a layer spec
    with a second norm but no feed-forward gets ``x <- norm(a * x)``.  The block
    carries ``(x in the activation type, x in 32-bit)``: sublayers read the first, the sums and norms
    the second (``ModelSpec.residual_stream = "float32"``).  The norms are parts with
    ``forward_stream`` (``parts.norm.LayerNorm``)."""

    def __init__(self, spec, dtype):
        self.spec = spec
        self.alpha = float(spec.residual_scale)
        self.mixer = make_mixer(spec.mixer, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
        if spec.feed_forward_norm is not None:      # without a feed-forward: the norm of a * x alone
            self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "forward_stream"):
                raise ValueError("a post-norm block needs norms that work on the 32-bit stream (forward_stream)")

    def parts(self) -> dict:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out["feed_forward"] = self.feed_forward
        if self.feed_forward_norm is not None:
            out["feed_forward_norm"] = self.feed_forward_norm
        return out

    def forward(self, hidden, stream, step, slot):
        y = self.mixer.forward(hidden, step, slot)
        hidden, stream = self.mixer_norm.forward_stream(stream, y, self.alpha)
        if self.feed_forward_norm is not None:
            y = self.feed_forward.forward(hidden, step) if self.feed_forward is not None else None
            hidden, stream = self.feed_forward_norm.forward_stream(stream, y, self.alpha)
        return hidden, stream


class PreNormStreamBlock:
    """Norm before each sublayer, over a 32-bit stream: ``x <- x + mixer(norm(x))``, then (if the layer
    has a feed-forward) ``x <- x + feed_forward(norm(x))``.  The block carries ``(pending, stream)``:
    ``pending`` is the last sublayer's output that the stream has not taken in yet (None at the
    start); the next norm call adds it in 32-bit and normalises the sum in one kernel.  Whoever
    needs the stream itself (the model's last norm, a tap, the start of a looped pass) adds
    ``pending`` first.  The norms are parts with ``forward_stream(stream, y)``
    (``parts.norm.RMSNorm``)."""

    def __init__(self, spec, dtype):
        self.spec = spec
        self.mixer = make_mixer(spec.mixer, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
            self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "forward_stream"):
                raise ValueError("a block over the 32-bit stream needs norms with forward_stream")

    def parts(self) -> dict:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out["feed_forward"] = self.feed_forward
            out["feed_forward_norm"] = self.feed_forward_norm
        return out

    def forward(self, pending, stream, step, slot):
        x, stream = self.mixer_norm.forward_stream(stream, pending)
        pending = self.mixer.forward(x, step, slot)
        if self.feed_forward is not None:
            x, stream = self.feed_forward_norm.forward_stream(stream, pending)
            pending = self.feed_forward.forward(x, step)
        return pending, stream


class SublayerNormBlock:
    """Norm on each sublayer's output, over a 32-bit stream: ``x <- x + norm(mixer(x))``, then (if the
    layer has a feed-forward) ``x <- x + norm(feed_forward(x))``.  The sublayers read ``x`` itself.  The
    block carries ``(x in the activation type, x in 32-bit)`` like :class:`PostNormBlock`
    (``ModelSpec.residual_stream = "float32"``); norm, add and the rounded copy are one kernel.  The norms
    are parts with ``forward_into_stream(stream, y)`` (``parts.norm.RMSNorm``)."""

    def __init__(self, spec, dtype):
        self.spec = spec
        self.mixer = make_mixer(spec.mixer, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
            self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not hasattr(n, "forward_into_stream"):
                raise ValueError("a block with norms on the sublayers' outputs needs norms with forward_into_stream")

    def parts(self) -> dict:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out["feed_forward"] = self.feed_forward
            out["feed_forward_norm"] = self.feed_forward_norm
        return out

    def forward(self, hidden, stream, step, slot):
        y = self.mixer.forward(hidden, step, slot)
        hidden, stream = self.mixer_norm.forward_into_stream(stream, y)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(hidden, step)
            hidden, stream = self.feed_forward_norm.forward_into_stream(stream, y)
        return hidden, stream


class StreamMixBlock:
    """Pre-norm over several 32-bit residual streams (``parts.streams``): every sublayer reads a learned
    mixture of the streams through its norm and writes its (optionally gated) result back into all of
    them.  The block carries ``(pending, streams)``: ``pending = (StreamMix, y, gate logits)`` is the last
    sublayer's result that the streams have not taken in yet (None at the start); the next sublayer's
    read applies it in the same kernel.  Whoever needs the streams themselves (the model's last norm, a
    tap) applies ``pending`` first.  The norms are RMS norms with a 32-bit weight."""

    def __init__(self, spec, dtype):
        from .streams import StreamMix
        self.spec = spec
        self.dtype = dtype
        self.mixer = make_mixer(spec.mixer, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        if "mixer_streams" not in spec.extra:
            raise ValueError("a stream_mix block needs extra['mixer_streams'] (a StreamMixSpec)")
        self.mixer_streams = StreamMix(spec.extra["mixer_streams"], dtype)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_streams = None
        if spec.feed_forward is not None:
            self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
            self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)
            if "feed_forward_streams" not in spec.extra:
                raise ValueError("a stream_mix block with a feed-forward needs extra['feed_forward_streams']")
            self.feed_forward_streams = StreamMix(spec.extra["feed_forward_streams"], dtype)

    def parts(self) -> dict:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "mixer_streams": self.mixer_streams}
        if self.feed_forward is not None:
            out.update({"feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm,
                        "feed_forward_streams": self.feed_forward_streams})
        return out

    @staticmethod
    def read(streams, pending, mix, norm, dtype):
        """Apply ``pending`` to the streams and read them for the sublayer whose numbers ``mix`` holds: the
        normed mixture in the activation type."""
        from ..csrc import ops
        h = torch.empty(streams.shape[0], streams.shape[2], dtype=dtype, device=streams.device)
        write = pending[0].write_args(pending[1], pending[2]) if pending is not None else None
        if norm.weight.dtype != torch.float32:
            raise ValueError("a stream_mix block needs norms with a 32-bit weight (RMSNormSpec.offset)")
        ops.stream_mix(streams, write=write, read=(mix.read_weights(streams.device), norm.weight, norm.spec.eps, h),
                       dtype=dtype)
        return h

    def sublayers(self):
        """(name, run(h, step, slot), StreamMix, norm) of each sublayer, in order."""
        out = [("mixer." + self.mixer.spec.kind, lambda h, step, slot: self.mixer.forward(h, step, slot),
                self.mixer_streams, self.mixer_norm)]
        if self.feed_forward is not None:
            out.append(("feed_forward." + self.feed_forward.spec.kind, lambda h, step, slot: self.feed_forward.forward(h, step),
                        self.feed_forward_streams, self.feed_forward_norm))
        return out

    def forward(self, pending, streams, step, slot, timed=None):
        run = timed if timed is not None else (lambda name, fn, *a: fn(*a))
        for name, sub, mix, norm in self.sublayers():
            h = run("stream_mix", self.read, streams, pending, mix, norm, self.dtype)
            y = run(name, sub, h, step, slot)
            pending = (mix, y, run("stream_gate", mix.gate_logits, h))
        return pending, streams


ARRANGEMENTS = {"stream_mix": StreamMixBlock, "pre_norm": PreNormBlock, "post_norm": PostNormBlock, "pre_norm_stream": PreNormStreamBlock,
                "sublayer_norm": SublayerNormBlock}


def make_block(spec, dtype):
    if spec.arrangement not in ARRANGEMENTS:
        raise ValueError(f"unknown block arrangement {spec.arrangement!r}; known: {sorted(ARRANGEMENTS)}")
    return ARRANGEMENTS[spec.arrangement](spec, dtype)
