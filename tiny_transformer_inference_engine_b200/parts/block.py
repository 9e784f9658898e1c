"""Arrangement of a layer's parts.

``pre_norm`` is the reference's block (models/transformer_block.py:149-158):
``x = x + mixer(norm1(x))``, ``x = x + ffn(norm2(x))``.  The sums are formed in the
32-bit residual stream by the norm kernels: a sub-layer's output waits in
``stream.delta`` and the next norm adds it while normalising.  A layer without a
feed-forward (``ffn`` None) has only the first sub-layer.
"""
from __future__ import annotations

from .base import Block, PartSpec, ResidualStream, StepContext, mixer_cache_argument
from ..registry import register_part, build_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, prefix: str, mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec = None, ffn: PartSpec = None):
        super().__init__(prefix)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.ffn_norm = build_part("norm", ffn_norm) if ffn is not None else None
        self.ffn = build_part("ffn", ffn) if ffn is not None else None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def cache_needs(self):
        return self.mixer.cache_needs()                            # the feed-forward parts here keep nothing between steps

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        h = self.mixer_norm.add_norm(stream.resid, stream.delta)
        a = self.mixer.forward(h, ctx, mixer_cache_argument(self.mixer, caches))
        if self.ffn is None:
            stream.delta = a
            return
        h = self.ffn_norm.add_norm(stream.resid, a)
        stream.delta = self.ffn.forward(h, ctx)


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """Post-norm: ``x = LN_a(alpha * x + mixer(x))`` followed by ``x = LN_b(alpha * x + ffn(x))``; each sub-layer's input is
    the (already normalised) stream, not a normed copy of it.  The stream holds ``x`` in 32-bit; each norm kernel forms the scaled sum, normalises, rewrites the
    stream and hands the next sub-layer a copy in the compute dtype.  A layer without a feed-forward (``ffn`` None) ends
    after the first norm."""

    def __init__(self, prefix: str, mixer: PartSpec, mixer_norm: PartSpec, ffn, ffn_norm, alpha: float = 1.0):
        super().__init__(prefix)
        self.alpha = float(alpha)
        self.mixer = build_part("mixer", mixer)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.ffn_norm = build_part("norm", ffn_norm) if ffn is not None else None

    def children(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        if stream.delta is not None:
            raise ValueError("a post-norm block cannot follow a block that leaves a sum unformed")
        x = stream.x
        if x is None:                                               # the first layer: the embedding's rows
            x = stream.resid if self.dtype == stream.resid.dtype else self.ops.cast_rows(stream.resid, self.dtype)
        a = self.mixer.forward(x, ctx, mixer_cache_argument(self.mixer, caches))
        x = self.mixer_norm.scale_add_norm(stream.resid, a, self.alpha)
        if self.ffn is not None:
            f = self.ffn.forward(x, ctx)
            x = self.ffn_norm.scale_add_norm(stream.resid, f, self.alpha)
        stream.x = x
