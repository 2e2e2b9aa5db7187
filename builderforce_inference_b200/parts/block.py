"""Residual blocks.  The residual stream stays float32 in every run dtype; the adds happen inside
the mixer's and the feed-forward's last matrix product.

``prenorm``   ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (crates/bfi-models/src/qwen3.rs:217-250).
``parallel``  one norm, both sublayers read its output: ``h = norm1(x); x += mixer(h) + ffn(h)``;
              the feed-forward may be absent.
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, PartSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec):
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.norm2 = NORMS.build(norm2)
        self.ffn = FEED_FORWARDS.build(ffn)

    def children(self):
        return {"norm1": self.norm1, "mixer": self._mixer, "norm2": self.norm2, "ffn": self.ffn}

    def mixer(self):
        return self._mixer

    def forward(self, ctx, residual, run) -> None:
        h = self.norm1.forward(ctx, residual)
        self._mixer.forward(ctx, h, residual, run)
        h = self.norm2.forward(ctx, residual)
        self.ffn.forward(ctx, h, residual)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    graph_safe = True

    def __init__(self, norm1: PartSpec, mixer: PartSpec, ffn: PartSpec = None):
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.ffn = FEED_FORWARDS.build(ffn) if ffn is not None else None

    def children(self):
        out = {"norm1": self.norm1, "mixer": self._mixer}
        if self.ffn is not None:
            out["ffn"] = self.ffn
        return out

    def mixer(self):
        return self._mixer

    def forward(self, ctx, residual, run) -> None:
        # neither sublayer reads the residual stream, so each may add its output as it is done
        h = self.norm1.forward(ctx, residual)
        self._mixer.forward(ctx, h, residual, run)
        if self.ffn is not None:
            self.ffn.forward(ctx, h, residual)
