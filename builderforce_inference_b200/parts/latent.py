"""Latent attention, as a mixer: keys and values of all heads are made from one small vector per
token, and only that vector is cached.

Per token with input ``h``: the queries ``q = W_q h``, head by head ``[dim unrotated | rot_dim
rotated]``; the down projection ``W_dkv h`` whose first ``kv_rank`` values, RMS-normed, are the
latent ``c`` and whose last ``rot_dim`` values are one rotated key part that all heads share.  Head
``a``'s unrotated key is ``W_uk_a c``, its value ``W_uv_a c``; its score against a token is
``(q_a^n . k_a^n + q_a^r . k^r) * scale``; the softmax is causal and may carry a learned sink per
head in its denominator; head ``a``'s output may be multiplied by ``sigmoid(W_g h)_a``; ``W_o`` acts
on the concatenated heads.

Here the attention runs in the latent space.  Since ``q_a^n . W_uk_a c = (W_uk_a^T q_a^n) . c`` and
``sum_j p_j W_uv_a c_j = W_uv_a sum_j p_j c_j``, every query head becomes
``[W_uk_a^T q_a^n | rot(q_a^r)]`` (``kv_rank + rot_dim`` values), all heads read the same cached
rows ``[c | rot(k^r)]`` as ONE key/value head whose values are the first ``kv_rank`` values of its
keys, and ``W_uv_a`` takes head ``a``'s weighted sum of latents to its ``v_dim`` outputs.  The cache
holds ``kv_rank + rot_dim`` values per token and nothing is expanded per cached token, whatever
the number of heads; a layer without a down projection of its own (``own_kv`` false) reads the
rows another layer's run has written, with its own ``W_uk`` and ``W_uv``.

Launches: one product for queries, gate logits and down projection together; ``latent_prepare``
(rotations, the latent's norm, the cache write); ``latent_absorb``; the attention (in bfloat16 the
tensor-core kernel over stacked (token, head) rows, cut into key ranges when a step has few rows;
otherwise the general paged kernel, and the gate then waits for ``latent_expand``);
``latent_expand`` (``W_uv`` and the gate); the output product, which adds into the residual stream.
In bfloat16 steps of more than ``PRODUCT_MIN_TOKENS`` tokens, ``latent_absorb`` and ``latent_expand``
are one tensor-core product per head each, on slices of the same buffers.

Further variants, each a parameter.  ``q_rank``: the queries go through a latent of their own,
``q = W_uq norm(W_dq h)`` (an RMS norm with a weight of ``q_rank`` values); the first product then
makes ``[gate | down projection | query latent]``, a norm kernel makes the normed query latent and a
second product the queries, into the columns the first one left free.  ``gate`` ``"value"``: one gate
per output value (``W_g`` has ``heads * v_dim`` rows) instead of one per head; it is applied where
``W_uv`` is.  A position encoding of the ``adjacent`` pairing (value 2i turns with value 2i + 1): a
score is a dot product over the rotated part, which does not change when the queries' and the
keys' rotated values are reordered alike, so at load the rows of the query and down projections
that make rotated values are reordered (even ones first, then odd ones) and the kernels rotate
with the ``half`` pairing; the cache then holds the reordered key part.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, linear
from .base import MIXERS, POSITION_ENCODINGS, KVNeed, Mixer, ParamSpec, PartSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    PRODUCT_MIN_TOKENS = 64     # steps of more tokens: W_uk^T and W_uv as one matrix product per head

    def __init__(self, width: int, n_heads: int, dim: int, rot_dim: int, v_dim: int, kv_rank: int,
                 position: Optional[PartSpec] = None, eps: float = 1e-6, scale: Optional[float] = None,
                 own_kv: bool = True, sink=None, gate=False, q_rank: Optional[int] = None):
        if n_heads < 1 or dim < 1 or rot_dim < 0 or v_dim < 1 or kv_rank < 1:
            raise ValueError(f"latent attention: bad sizes heads={n_heads} dim={dim} rot_dim={rot_dim} v_dim={v_dim} "
                             f"kv_rank={kv_rank}")
        if (kv_rank + rot_dim) % 2 != 0 or kv_rank + rot_dim > 1024 or kv_rank > 512:
            raise ValueError(f"latent attention: kv_rank = {kv_rank} must be at most 512, kv_rank + rot_dim = "
                             f"{kv_rank + rot_dim} even and at most 1024")
        if not (sink is None or sink == "learned" or isinstance(sink, (int, float))):
            raise ValueError(f"sink must be a number or 'learned', got {sink!r}")
        self.width, self.n_heads, self.dim, self.rot_dim = int(width), int(n_heads), int(dim), int(rot_dim)
        self.v_dim, self.kv_rank, self.eps = int(v_dim), int(kv_rank), float(eps)
        self.scale = float(scale) if scale is not None else (dim + rot_dim) ** -0.5
        if gate not in (False, None, True, "head", "value"):
            raise ValueError(f"gate must be false, 'head' or 'value', got {gate!r}")
        if q_rank is not None and q_rank < 1:
            raise ValueError(f"latent attention: bad size q_rank={q_rank}")
        self.own_kv, self.has_gate = bool(own_kv), bool(gate)
        self.gate_values = gate == "value" and v_dim > 1      # with values of one number a gate per value is a gate per head
        self.q_rank = None if q_rank is None else int(q_rank)
        self.learned_sink = sink == "learned"
        self.sink = None if sink is None or self.learned_sink else float(sink)
        self.position = POSITION_ENCODINGS.build(position) if position is not None \
            else POSITION_ENCODINGS.build(PartSpec("none"))
        rot_used = getattr(self.position, "rot_dim", 0)
        if rot_used > self.rot_dim:
            raise ValueError(f"latent attention: {rot_used} rotated values do not fit a rotated part of {self.rot_dim}")
        self.rot_used = rot_used
        self.reorder = getattr(self.position, "pairing", "half") == "adjacent"

    def children(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        w, a = self.width, self.n_heads
        specs = {"uk_proj": ParamSpec((a * self.dim, self.kv_rank)),
                 "uv_proj": ParamSpec((a * self.v_dim, self.kv_rank)),
                 "o_proj": ParamSpec((w, a * self.v_dim))}
        if self.own_kv:
            specs["dkv_proj"] = ParamSpec((self.kv_rank + self.rot_dim, w))
            specs["dkv_norm"] = ParamSpec((self.kv_rank,), "norm")
        if self.q_rank is None:
            specs["q_proj"] = ParamSpec((a * (self.dim + self.rot_dim), w))
        else:
            specs.update({"dq_proj": ParamSpec((self.q_rank, w)), "dq_norm": ParamSpec((self.q_rank,), "norm"),
                          "uq_proj": ParamSpec((a * (self.dim + self.rot_dim), self.q_rank))})
        if self.learned_sink:
            specs["sink"] = ParamSpec((a,), "matrix")
        if self.has_gate:
            specs["g_proj"] = ParamSpec((a * self.v_dim if self.gate_values else a, w))
        return specs

    def cache_need(self):
        return KVNeed(1, self.kv_rank + self.rot_dim, v_dim=self.kv_rank, values_in_keys=True)

    def prepare(self, runtime, max_positions: int) -> None:
        self.position.prepare(runtime, max_positions)

    def _reordered(self, m: torch.Tensor, first: int, stride: int, count: int) -> torch.Tensor:
        """``m`` with the rows ``first + i * stride + (0 .. rot_used)`` for ``i < count`` reordered from
        adjacent pairs to halves: the even ones, then the odd ones."""
        if not self.reorder or self.rot_used < 2:
            return m
        idx = torch.arange(m.shape[0], device=m.device)
        order = torch.cat([torch.arange(0, self.rot_used, 2), torch.arange(1, self.rot_used, 2)]).to(m.device)
        for i in range(count):
            at = first + i * stride
            idx[at:at + self.rot_used] = at + order
        return m.index_select(0, idx)

    def load(self, tensors, runtime) -> None:
        # one product makes the queries (or, with a query latent, leaves room for them), the gate logits, the
        # down projection and the query latent: rows in that order, each part starting on 16 bytes
        a, dq = self.n_heads, self.dim + self.rot_dim
        q_cols = a * dq
        parts, at = [], 0

        def put(m):
            nonlocal at
            pad = (-at) % 8
            if pad:
                parts.append(torch.zeros((pad, self.width), dtype=m.dtype, device=m.device))
                at += pad
            start = at
            parts.append(m)
            at += m.shape[0]
            return start

        if self.q_rank is None:
            put(self._reordered(tensors["q_proj"], self.dim, dq, a))
            self.first_col = 0
        else:
            self.first_col = at = q_cols + (-q_cols) % 8     # the first product writes behind the queries' columns
            self.w_uq = self._reordered(tensors["uq_proj"], self.dim, dq, a).contiguous()
            self.dq_norm = tensors["dq_norm"].contiguous()
        self.gate_off = self.kv_off = self.cq_off = at
        if self.has_gate:
            self.gate_off = put(tensors["g_proj"]) if self.q_rank is not None else at
            if self.q_rank is None:          # directly behind the queries, as the kernels have always found it
                parts.append(tensors["g_proj"])
                at += tensors["g_proj"].shape[0]
        if self.own_kv:
            self.kv_off = put(self._reordered(tensors["dkv_proj"], self.kv_rank, 0, 1))
        if self.q_rank is not None:
            self.cq_off = put(tensors["dq_proj"])
        self.n_cols = at
        if len({m.dtype for m in parts}) > 1:
            parts = [m.float() for m in parts]
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]
        self.w_uk = tensors["uk_proj"].contiguous()
        self.w_uv = tensors["uv_proj"].contiguous()
        # steps of many tokens take W_uk^T and W_uv to the tensor cores head by head: W_uk_a^T as a
        # matrix of its own ([kv_rank, dim]), when every slice starts on 16 bytes
        sizes = (self.dim, self.dim + self.rot_dim, self.kv_rank, self.kv_rank + self.rot_dim, self.v_dim, self.n_cols)
        self.w_uk_t = None
        if self.w_uk.dtype == torch.bfloat16 and all(n % 8 == 0 for n in sizes):
            self.w_uk_t = self.w_uk.view(self.n_heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_o = tensors["o_proj"]
        self.dkv_norm = tensors["dkv_norm"].contiguous() if self.own_kv else None
        self.sinks = tensors["sink"].float().contiguous() if self.learned_sink else None
        if self.sink is not None:          # one number for all heads: the tensor-core kernel reads one per head
            self.sinks = torch.full((self.n_heads,), self.sink, dtype=torch.float32, device=self.w_uk.device)

    def forward(self, ctx, h, residual, run) -> None:
        self._run(ctx, h, residual, run, EPI_ACCUMULATE)

    def forward_store(self, ctx, h, out, run) -> None:
        self._run(ctx, h, out, run, EPI_STORE)

    def _run(self, ctx, h, target, run, epilogue) -> None:
        kv = run.kv
        if kv is None:
            raise RuntimeError("latent attention needs a cache for its run")
        if run.writes_cache != self.own_kv:
            raise RuntimeError("a latent attention layer writes the cache exactly when it has a down projection")
        a, r, rd = self.n_heads, self.kv_rank, self.rot_dim
        proj = ctx.rows("latent.proj", self.n_cols)
        if self.q_rank is None:
            linear(h, self.w_in, proj, EPI_STORE)
        else:
            linear(h, self.w_in, proj[:, self.first_col:], EPI_STORE)
            cq = ctx.rows("latent.cq", self.q_rank)
            ops.rmsnorm(proj[:, self.cq_off:self.cq_off + self.q_rank], self.dq_norm, self.eps, cq)
            linear(cq, self.w_uq, proj[:, :a * (self.dim + rd)], EPI_STORE)
        table, rot_used = self.position.fused_rotary()
        qa = ctx.rows("latent.q", a * (r + rd))
        ops.latent_prepare(proj, qa, a, self.dim, rd, r, self.kv_off, self.dkv_norm, self.eps, table, rot_used,
                           ctx.token_pos, ctx.token_slot, kv, run.writes_cache, ctx.status)
        products = self.w_uk_t is not None and proj.dtype == torch.bfloat16 and ctx.n_tokens > self.PRODUCT_MIN_TOKENS
        if products:
            dq = self.dim + rd
            for i in range(a):
                linear(proj[:, i * dq:i * dq + self.dim], self.w_uk_t[i], qa[:, i * (r + rd):i * (r + rd) + r], EPI_STORE)
        else:
            ops.latent_absorb(proj, self.w_uk, qa, ctx.token_slot, a, self.dim, rd, r)
        lat = ctx.rows("latent.out", a * r)
        n_gate = a * self.v_dim if self.gate_values else a
        gate = proj[:, self.gate_off:self.gate_off + n_gate] if self.has_gate else None
        if self.attend(ctx, qa, lat, kv, None if self.gate_values else gate):
            gate = None                    # the attention has applied it
        out = ctx.rows("attn.out", a * self.v_dim)
        if products and (gate is None or self.gate_values):
            dv = self.v_dim
            for i in range(a):
                linear(lat[:, i * r:(i + 1) * r], self.w_uv[i * dv:(i + 1) * dv], out[:, i * dv:(i + 1) * dv], EPI_STORE)
            if gate is not None:
                ops.sigmoid_gate(out, gate, 1)
        else:
            ops.latent_expand(lat, self.w_uv, gate, out, ctx.token_slot, a, self.v_dim, r)
        linear(out, self.w_o, target, epilogue)

    def attend(self, ctx, qa, lat, kv, gate=None) -> bool:
        """The attention in the latent space; True if it has multiplied the heads' outputs by their
        gates (a scalar per token and head, so it commutes with ``W_uv``)."""
        if qa.dtype == torch.bfloat16:
            from ..kernels import fast_ops
            if fast_ops.attention_latent_bf16(ctx, qa, lat, kv, self.n_heads, self.scale, self.sinks, gate=gate):
                return gate is not None
        sink = self.sinks if self.learned_sink else self.sink
        ops.attention_paged(qa, qa.stride(0), lat, kv, ctx.cu_seqlens, ctx.seq_slot, ctx.seq_start,
                            ctx.n_seqs, ctx.max_seq_tokens, self.n_heads, self.scale, sink)
        return False
