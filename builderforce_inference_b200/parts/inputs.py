"""Parts that add to the embedded tokens before the first block.

``hashed_bigram``: a second embedding that depends on the token and the one before it:
``x[t] += table[(token[t-1] * mul_prev + token[t] * mul_cur) mod buckets]``; a sequence's first
token, which has no predecessor, takes the table's last row (number ``buckets``), so the table has
``buckets + 1`` rows.  The predecessor of the first token a step brings for a sequence was the
last token of an earlier step: it is kept per sequence (one int32 per slot, beside the mixers'
fixed-size states) and moved on after every step, so a prompt may arrive in pieces and decoding
goes on token by token with the same result.  Both kernels read the step's device arrays only,
so the part is graph-safe.
"""
from __future__ import annotations

from typing import Dict

from ..kernels import ops
from .base import INPUT_PARTS, InputPart, ParamSpec, StateNeed


@INPUT_PARTS.register("hashed_bigram")
class HashedBigram(InputPart):
    graph_safe = True

    def __init__(self, width: int, vocab: int, buckets: int, mul_prev: int, mul_cur: int):
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"hashed bigram: {buckets} buckets, multipliers {mul_prev} and {mul_cur}")
        # the hash is evaluated in 64-bit integers
        if (vocab - 1) * (int(mul_prev) + int(mul_cur)) >= 2 ** 62:
            raise ValueError("hashed bigram: the multipliers are too large for the vocabulary")
        self.width, self.vocab, self.buckets = int(width), int(vocab), int(buckets)
        self.mul_prev, self.mul_cur = int(mul_prev), int(mul_cur)
        self.table = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.buckets + 1, self.width), "table")}

    def cache_need(self):
        return StateNeed((1,), "int32")

    def load(self, tensors, runtime) -> None:
        self.table = tensors["table"].contiguous()

    def forward(self, ctx, x, run) -> None:
        last = run.state
        if last is None:
            raise RuntimeError("the hashed bigram embedding needs its per-sequence state")
        ops.bigram_add(self.table, ctx.token_ids, ctx.token_pos, ctx.token_slot, last, x, self.mul_prev, self.mul_cur,
                       self.vocab, ctx.status)
        ops.keep_last_tokens(ctx.token_ids, ctx.cu_seqlens, ctx.seq_slot, last, ctx.n_seqs)
