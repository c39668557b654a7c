"""Residual blocks.  The residual stream stays float32 in every run dtype; the adds happen inside
the mixer's and the feed-forward's last matrix product.

``prenorm``   ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (crates/bfi-models/src/qwen3.rs:217-250); the
              feed-forward (with its norm) may be absent.
``parallel``  one norm, both sublayers read its output: ``h = norm1(x); x += mixer(h) + ffn(h)``;
              the feed-forward may be absent.
``sandwich``  a norm before and after each sublayer: ``x += norm1b(mixer(norm1(x)));
              x += norm2b(ffn(norm2(x)))``; the feed-forward (with its two norms) may be absent.
              The sublayers write their output to a float32 buffer (``forward_store``) and the
              second norm adds it, normed, into the residual stream in one kernel, which also makes
              the feed-forward's input norm.
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, PartSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec = None, ffn: PartSpec = None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("a pre-norm block has a feed-forward with its norm, or neither")
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.norm2 = NORMS.build(norm2) if ffn is not None else None
        self.ffn = FEED_FORWARDS.build(ffn) if ffn is not None else None

    def children(self):
        out = {"norm1": self.norm1, "mixer": self._mixer}
        if self.ffn is not None:
            out.update({"norm2": self.norm2, "ffn": self.ffn})
        return out

    def mixer(self):
        return self._mixer

    def forward(self, ctx, residual, run) -> None:
        h = self.norm1.forward(ctx, residual)
        self._mixer.forward(ctx, h, residual, run)
        if self.ffn is None:
            return
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


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    graph_safe = True

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm1b: PartSpec, norm2: PartSpec = None,
                 ffn: PartSpec = None, norm2b: PartSpec = None):
        if (ffn is None) != (norm2 is None) or (ffn is None) != (norm2b is None):
            raise ValueError("a sandwich block has a feed-forward with both of its norms, or none of the three")
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.norm1b = NORMS.build(norm1b)
        self.norm2 = NORMS.build(norm2) if ffn is not None else None
        self.ffn = FEED_FORWARDS.build(ffn) if ffn is not None else None
        self.norm2b = NORMS.build(norm2b) if ffn is not None else None

    def children(self):
        out = {"norm1": self.norm1, "mixer": self._mixer, "norm1b": self.norm1b}
        if self.ffn is not None:
            out.update({"norm2": self.norm2, "ffn": self.ffn, "norm2b": self.norm2b})
        return out

    def mixer(self):
        return self._mixer

    def forward(self, ctx, residual, run) -> None:
        import torch
        y = ctx.rows("sublayer.out", residual.shape[1], torch.float32)
        h = self.norm1.forward(ctx, residual)
        self._mixer.forward_store(ctx, h, y, run)
        if self.ffn is None:
            self.norm1b.add_to(ctx, residual, y)
            return
        h = self.norm1b.add_to(ctx, residual, y, then=self.norm2)      # the add and the next norm in one kernel
        self.ffn.forward_store(ctx, h, y)
        self.norm2b.add_to(ctx, residual, y)
