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
``outnorm``   a norm on each sublayer's OUTPUT only; the sublayers read the residual stream itself:
              ``x += mult * norm1(g1 * mixer(c1(x))); x += mult * norm2(g2 * ffn(c2(x)))``.  ``c`` is the
              identity or, with ``conv_taps``, ``c(x)_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j)``, a
              causal convolution over time per channel whose last ``taps - 1`` inputs are kept per
              sequence (the block asks the cache for them beside what its mixer keeps); ``g`` is 1 or,
              with ``gate``, ``sigmoid(W_g x + b_g)`` element by element, made from the residual stream
              as it stands before the convolution.  One kernel reads the float32 stream and writes
              both the convolved and the plain copy in the activation dtype; one kernel gates, norms,
              scales and adds the sublayer's float32 output.  In steps in which every sequence
              brings one token that kernel also makes the input of the sublayer that follows (the next
              convolution, of this block or of the out-norm block that runs next) from the row it has
              just written, so a sublayer costs one launch around it instead of two.  The feed-forward
              (with its norm, convolution and gate) may be absent.
"""
from __future__ import annotations

from typing import Dict

from ..cache.cache import KVView, RunCache, needs_of
from ..kernels import ops
from ..kernels.linear import EPI_STORE, linear
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, ParamSpec, PartSpec, StateNeed


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


@BLOCKS.register("outnorm")
class OutNormBlock(Block):
    graph_safe = True

    def __init__(self, width: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec = None, ffn: PartSpec = None,
                 mult: float = 1.0, conv_taps: int = None, gate: bool = False):
        if (ffn is None) != (norm2 is None):
            raise ValueError("an out-norm block has a feed-forward with its norm, or neither")
        if conv_taps is not None and not 1 <= conv_taps <= 16:
            raise ValueError(f"an out-norm block's input convolution takes 1 to 16 taps, got {conv_taps}")
        self.width, self.mult = int(width), float(mult)
        self.taps = None if conv_taps is None else int(conv_taps)
        self.has_gate = bool(gate)
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.norm2 = NORMS.build(norm2) if ffn is not None else None
        self.ffn = FEED_FORWARDS.build(ffn) if ffn is not None else None
        self.n_sub = 1 if self.ffn is None else 2
        self.conv_w = [None, None]
        self.gate_w = [None, None]
        self.gate_b = [None, None]
        self.no_history = None

    def children(self):
        out = {"norm1": self.norm1, "mixer": self._mixer}
        if self.ffn is not None:
            out.update({"norm2": self.norm2, "ffn": self.ffn})
        return out

    def mixer(self):
        return self._mixer

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {}
        for i in range(1, self.n_sub + 1):
            if self.taps is not None:
                specs[f"conv{i}"] = ParamSpec((self.width, self.taps))
            if self.has_gate:
                specs[f"gate{i}_proj"] = ParamSpec((self.width, self.width))
                specs[f"gate{i}_proj.bias"] = ParamSpec((self.width,))
        return specs

    def load(self, tensors, runtime) -> None:
        for i in range(self.n_sub):
            if self.taps is not None:
                self.conv_w[i] = tensors[f"conv{i + 1}"].contiguous()
            if self.has_gate:
                self.gate_w[i] = tensors[f"gate{i + 1}_proj"]
                self.gate_b[i] = tensors[f"gate{i + 1}_proj.bias"].contiguous()
        import torch
        self.no_history = torch.empty((1, 0, self.width), dtype=torch.float32, device=runtime.device)

    def _own_needs(self) -> tuple:
        if self.taps is None or self.taps == 1:
            return ()
        return (StateNeed((self.taps - 1, self.width), "float32"),) * self.n_sub

    def cache_need(self):
        return needs_of(self._mixer.cache_need()) + self._own_needs()

    def _input(self, ctx, x, i: int, kept):
        """What sublayer ``i`` reads (convolved) and what its gate reads (plain), in the activation dtype."""
        h = ctx.rows("block.in", self.width)
        plain = ctx.rows("block.plain", self.width) if self.has_gate else None
        if self.taps is None:
            h.copy_(x)
            return h, h
        single = ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs
        ops.causal_conv(x, 0, self.width, self.conv_w[i], None, kept, h, ctx.token_slot, ctx.cu_seqlens, ctx.seq_slot,
                        ctx.n_seqs, single_tokens=single, act=ops.CONV_ACT_NONE, add_input=True, copy=plain)
        return h, plain

    def _output(self, ctx, x, y, plain, i: int, norm, follow=None):
        """The sublayer's output into the stream.  ``follow`` ``(weights, kept inputs)``: the convolution
        in front of the sublayer that runs next, made in the same kernel; returns its two outputs."""
        glog = None
        if self.has_gate:
            glog = ctx.rows("block.gate", self.width)
            linear(plain, self.gate_w[i], glog, EPI_STORE)
        conv = made = None
        if follow is not None:
            made = (ctx.rows("block.in", self.width), ctx.rows("block.plain", self.width))
            conv = (follow[0], follow[1], ctx.token_slot) + made
        norm.add_to(ctx, x, y, mult=self.mult, gate=glog, gate_bias=self.gate_b[i], conv=conv)
        return made

    def follows_in_one_kernel(self, ctx) -> bool:
        """Whether the convolution in front of this block's sublayers can ride on the kernel behind the
        sublayer before: single-token steps, 2 to 4 taps, rows in whole groups of 8 values, a gate."""
        return self.has_gate and self.taps is not None and 2 <= self.taps <= 4 and self.width % 8 == 0 \
            and ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs

    def _kept(self, run) -> list:
        own = self._own_needs()
        return list(run.entries[len(run.entries) - len(own):]) if own else [self.no_history] * self.n_sub

    def forward(self, ctx, residual, run) -> None:
        import torch
        if not run.writes_cache:
            raise RuntimeError("an out-norm block keeps its convolutions' inputs: its run needs a cache of its own")
        n_mixer = len(run.entries) - len(self._own_needs())
        entries = tuple(run.entries[:n_mixer])
        kept = self._kept(run)
        kv = next((e for e in entries if isinstance(e, KVView)), None)
        state = next((e for e in entries if not isinstance(e, KVView)), None)
        mixer_run = RunCache(kv=kv, state=state, writes_cache=True, entries=entries)
        y = ctx.rows("sublayer.out", self.width, torch.float32)
        fused = self.follows_in_one_kernel(ctx)
        # what the run after this one is, when it is an out-norm block of the same width: its first input is made here
        after = ctx.extras.get("next_block")
        after_run = ctx.extras.get("next_run")
        to_next = None
        if fused and isinstance(after, OutNormBlock) and after is not self and after.width == self.width \
                and after.follows_in_one_kernel(ctx) and after_run is not None and after_run.writes_cache:
            to_next = (after.conv_w[0], after._kept(after_run)[0])
        made = ctx.extras.pop("outnorm.input", None)
        if made is not None and made[0] is self:
            h, plain = made[1]
        else:
            h, plain = self._input(ctx, residual, 0, kept[0])
        self._mixer.forward_store(ctx, h, y, mixer_run)
        if self.ffn is None:
            made = self._output(ctx, residual, y, plain, 0, self.norm1, follow=to_next)
        else:
            made = self._output(ctx, residual, y, plain, 0, self.norm1, follow=(self.conv_w[1], kept[1]) if fused else None)
            h, plain = made if made is not None else self._input(ctx, residual, 1, kept[1])
            self.ffn.forward_store(ctx, h, y)
            made = self._output(ctx, residual, y, plain, 1, self.norm2, follow=to_next)
        if to_next is not None:
            ctx.extras["outnorm.input"] = (after, made)
