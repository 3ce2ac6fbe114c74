"""Arrangements of one layer: pre-norm mixer and feed-forward in sequence on a deferred residual, or side
by side on a 32-bit stream.

As the reference's decoder layer (kvcore/model/models/llama3.py:124-142): the running
``residual`` and the last sub-layer output ``h`` stay separate and are summed inside the
next norm; the first block starts with ``residual = h``.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import LayerSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Summed, WeightSlot


class PreNormResidualBlock(Block):
    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.mixer_norm = NORMS.build(layer.norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward_norm = NORMS.build(layer.norms["feed_forward_norm"], dtype=dtype, device=device)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def weight_slots(self) -> list[WeightSlot]:
        slots: list[WeightSlot] = []
        for part in self.parts():
            slots += part.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        names: list[str] = []
        for part in self.parts():
            names += part.ignorable_tensor_names()
        return names

    def finalize_weights(self) -> None:
        for part in self.parts():
            part.finalize_weights()

    def forward(self, h, residual, ctx, cache):
        # A part that can take its input before the norm (and fold the norm into its first matrix
        # product, the residual sum into its last) gets it that way; otherwise the norm runs as a
        # step of its own.  ``h`` may be ``Summed``: the part in front added its output already.
        scale, prenorm = self.mixer_norm.as_rms_scale(), getattr(self.mixer, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            a, residual = prenorm(h, residual, scale, ctx, cache)
        else:
            if isinstance(h, Summed):
                x = self.mixer_norm.forward(residual)
            elif residual is None:
                residual = h
                x = self.mixer_norm.forward(h)
            else:
                x, residual = self.mixer_norm.forward_residual(h, residual)
            a = self.mixer.forward(x, ctx, cache)
        scale, prenorm = self.feed_forward_norm.as_rms_scale(), getattr(self.feed_forward, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            h, residual = prenorm(a, residual, scale, ctx)
        else:
            if isinstance(a, Summed):
                x = self.feed_forward_norm.forward(residual)
            else:
                x, residual = self.feed_forward_norm.forward_residual(a, residual)
            h = self.feed_forward.forward(x, ctx)
        return h, residual


class ParallelResidualBlock(Block):
    """Mixer and feed-forward side by side on one stream: ``x <- x + (mixer(norm_a(x)) + ff(norm_b(x)))``,
    both norms reading the same ``x``.  The stream ``x`` is kept in 32-bit whatever the activation type:
    the two sub-layer outputs are added to each other and then to the stream in 32-bit by one kernel.
    A layer without a feed-forward (``layer.feed_forward is None``) adds the mixer alone.

    In the ``(h, residual)`` pair that runs through the blocks this block returns ``(Summed, stream)``."""

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.mixer_norm = NORMS.build(layer.norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(layer.norms["feed_forward_norm"], dtype=dtype, device=device)
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                     if p is not None)

    graph_safe = PreNormResidualBlock.graph_safe
    weight_slots = PreNormResidualBlock.weight_slots
    ignorable_tensor_names = PreNormResidualBlock.ignorable_tensor_names
    finalize_weights = PreNormResidualBlock.finalize_weights

    def forward(self, h, residual, ctx, cache):
        if residual is None:                       # the embedded tokens start the stream
            stream = K.stream_add(h)
        else:
            stream = residual if residual.dtype == torch.float32 else K.stream_add(residual)
            if not isinstance(h, Summed):          # a block in front left its last output unsummed
                stream = K.stream_add(stream, h)
        # Both sub-layers read the same stream, so a feed-forward that has something to get ready (a
        # ``prepare(x, ctx)`` whose result ``forward`` takes: a router whose grouping the host must see)
        # does that ahead of the mixer's launches, and nothing waits for it later.
        fx = prepared = None
        if self.feed_forward is not None:
            fx = self.feed_forward_norm.forward(stream)
            prepare = getattr(self.feed_forward, "prepare", None)
            prepared = None if prepare is None else prepare(fx, ctx)
        a = self.mixer.forward(self.mixer_norm.forward(stream), ctx, cache)
        f = None
        if self.feed_forward is not None:
            f = (self.feed_forward.forward(fx, ctx) if prepared is None
                 else self.feed_forward.forward(fx, ctx, prepared))
        return Summed(None), K.stream_add(stream, a, f)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
BLOCKS.register("parallel_residual", ParallelResidualBlock)

__all__ = ["ParallelResidualBlock", "PreNormResidualBlock"]
