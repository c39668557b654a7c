"""Mixers that keep a matrix state per head whose decay depends on the token.

Both run the same recurrence (``kernels/ops.decay_scan``): per head, with q_t, k_t of ``dim`` values
and v_t of ``vdim`` values,

    S_t = diag(a_t) S_(t-1) + k_t (c_t v_t)^T        o_t = S_t^T q_t + skip * v_t

and differ in where a_t and c_t come from and in what stands around the recurrence.  The state is
float32, zero when a slot is taken (the cache clears it), and, with the convolution's last inputs
where there is one, the only thing a sequence keeps: a step may bring whole prompts, further
pieces of one, or single tokens.  The decay, the step size and everything else that enters the
recurrence beside the projected q, k, v is evaluated in float32 inside the kernel.

``state_space`` (Mamba-2, state-space duality).  One input projection, laid out
``[z: inner | x: inner | B: groups*state | C: groups*state | dt: heads]`` with ``inner = heads * vdim``.
x, B and C together pass a causal convolution per channel (``conv_taps`` taps, with bias) and silu.
``dt = softplus(dt + dt_bias)``; head h (of group ``h // (heads/groups)``) runs the recurrence with
``k = B``, ``q = C``, ``v = x``, ``c = dt``, ``a = exp(-exp(A_log_h) dt)`` for all rows and ``skip = D_h``.
The output is multiplied by ``silu(z)``, then normed in ``norm_groups`` equal parts (weight ``norm``
over the whole row), then projected.

``gated_linear`` (gated linear attention).  ``q = W_q h * dim^(-1/2)``, ``k = W_k h``, ``v = W_v h``;
a decay per key channel ``a = sigmoid(W_a2 (W_a1 h) + b_a2)^(1/tau)``, ``c = 1``, no skip.  Every
head's output is normed over ``vdim`` (one weight of ``vdim`` values for all heads), multiplied by
``silu(W_g h)`` and projected.

``min_gru`` keeps ONE value per channel instead of a matrix per head (``kernels/ops.gated_scan``): with
``z = sigmoid(W_z h + b_z)`` and ``u = W_x h + b_x`` of ``inner`` values each,

    S_t = (1 - z_t) S_(t-1) + z_t cand(u_t)        out_t = W_o (S_t * silu(W_g h_t))

where ``cand(u) = u + 1/2`` for ``u >= 0`` and ``sigmoid(u)`` below (``candidate="positive"``), or ``u``
itself (``"identity"``).  Its gates read the current token only, so the recurrence is linear in S
and the kernel cuts a sequence's tokens into segments that run side by side.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, linear
from .base import MIXERS, Mixer, ParamSpec, StateNeed


CHUNK_TOKENS = 64            # chunk length of the chunked recurrence
CHUNKED_MIN_TOKENS = 192     # a step whose longest piece is shorter walks its tokens in order


def _as_f32(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


def _chunking(ctx, per_chunk: int, per_decay: int) -> dict:
    """The chunked form's arguments for a step with long pieces (none for short steps and single
    tokens): its scratch comes from the step's workspace."""
    if ctx.max_seq_tokens < CHUNKED_MIN_TOKENS:
        return {}
    n_chunks = ctx.n_tokens // CHUNK_TOKENS + ctx.n_seqs
    return {"chunk_len": CHUNK_TOKENS, "max_chunks": (ctx.max_seq_tokens + CHUNK_TOKENS - 1) // CHUNK_TOKENS,
            "chunk_state": ctx.rows("rec.chunk_state", per_chunk, torch.float32, n_rows=n_chunks),
            "chunk_decay": ctx.rows("rec.chunk_decay", per_decay, torch.float32, n_rows=n_chunks)}


@MIXERS.register("state_space")
class StateSpaceMixer(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, vdim: int, state: int, groups: int = 1, conv_taps: int = 4,
                 norm_groups: int = 1, eps: float = 1e-6):
        if n_heads < 1 or vdim < 1 or state < 1:
            raise ValueError(f"state-space mixer: bad sizes heads={n_heads} vdim={vdim} state={state}")
        if groups < 1 or n_heads % groups != 0:
            raise ValueError(f"state-space mixer: {n_heads} heads do not divide into {groups} groups")
        if norm_groups < 1 or (n_heads * vdim) % norm_groups != 0:
            raise ValueError(f"state-space mixer: {n_heads * vdim} values do not cut into {norm_groups} equal parts")
        if not 1 <= conv_taps <= 16:
            raise ValueError(f"state-space mixer: the convolution takes 1 to 16 taps, got {conv_taps}")
        self.width, self.n_heads, self.vdim, self.state, self.groups = int(width), int(n_heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(conv_taps), int(norm_groups), float(eps)
        self.inner = self.n_heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.state

    def param_specs(self) -> Dict[str, ParamSpec]:
        w = self.width
        return {"in_proj": ParamSpec((2 * self.inner + 2 * self.groups * self.state + self.n_heads, w)),
                "conv": ParamSpec((self.channels, self.taps)), "conv.bias": ParamSpec((self.channels,)),
                "dt_bias": ParamSpec((self.n_heads,)), "A_log": ParamSpec((self.n_heads,)),
                "D": ParamSpec((self.n_heads,), "norm"), "norm": ParamSpec((self.inner,), "norm"),
                "o_proj": ParamSpec((w, self.inner))}

    def cache_need(self):
        need = (StateNeed((self.n_heads, self.state, self.vdim), "float32"),)
        if self.taps > 1:
            need += (StateNeed((self.taps - 1, self.channels), "float32"),)
        return need

    def load(self, tensors, runtime) -> None:
        self.w_in, self.w_o = tensors["in_proj"], tensors["o_proj"]
        self.conv_w, self.conv_b = tensors["conv"], tensors["conv.bias"]
        if self.conv_w.dtype != self.conv_b.dtype:
            self.conv_w, self.conv_b = self.conv_w.float(), self.conv_b.float()
        self.norm = tensors["norm"]
        # the recurrence's constants, float32: the step's bias, the rate exp(A_log) and the skip factor
        self.dt_bias = _as_f32(tensors["dt_bias"])
        self.rate = torch.exp(_as_f32(tensors["A_log"]))
        self.skip = _as_f32(tensors["D"])
        self.no_history = torch.empty((1, 0, self.channels), dtype=torch.float32, device=runtime.device)

    def forward(self, ctx, h, residual, run) -> None:
        self._run(ctx, h, residual, run, EPI_ACCUMULATE)

    def forward_store(self, ctx, h, out, run) -> None:
        self._run(ctx, h, out, run, EPI_STORE)

    def _run(self, ctx, h, target, run, epilogue) -> None:
        if not run.writes_cache or len(run.entries) < (2 if self.taps > 1 else 1):
            raise RuntimeError("a state-space mixer needs a state of its own for its run")
        state = run.entries[0]
        inner, gn = self.inner, self.groups * self.state
        proj = ctx.rows("ssm.proj", 2 * inner + 2 * gn + self.n_heads)
        linear(h, self.w_in, proj, EPI_STORE)
        single = ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs
        xbc = ctx.rows("ssm.xbc", self.channels)
        kept = run.entries[1] if self.taps > 1 else self.no_history      # one tap: a factor and a bias, nothing is kept
        ops.causal_conv(proj, inner, self.channels, self.conv_w, self.conv_b, kept, xbc, ctx.token_slot,
                        ctx.cu_seqlens, ctx.seq_slot, ctx.n_seqs, single_tokens=single)
        y = ctx.rows("ssm.y", inner, torch.float32)
        ops.decay_scan(xbc, inner + gn, inner, xbc, 0, proj, 2 * inner + 2 * gn, y, state, ctx.cu_seqlens, ctx.seq_slot,
                       ctx.n_seqs, self.n_heads, self.state, self.vdim, self.n_heads // self.groups, ops.DECAY_STEP,
                       self.dt_bias, rate=self.rate, skip=self.skip, few_tokens=ctx.max_seq_tokens == 1, single_tokens=single,
                       **_chunking(ctx, self.n_heads * self.state * self.vdim, self.n_heads * self.state))
        g = ctx.rows("ssm.gated", inner)
        ops.gated_group_norm(y, proj[:, :inner], self.norm, self.eps, g, self.norm_groups, gate_first=True)
        linear(g, self.w_o, target, epilogue)


@MIXERS.register("gated_linear")
class GatedLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, tau: float, decay_rank: int = None,
                 eps: float = 1e-6):
        """``decay_rank`` (the width between the decay's two projections) may be left to the
        checkpoint: it is then the first size of ``a1_proj``."""
        decay_rank = -1 if decay_rank is None else int(decay_rank)
        if n_heads < 1 or dim < 1 or vdim < 1 or decay_rank == 0 or decay_rank < -1:
            raise ValueError(f"gated linear attention: bad sizes heads={n_heads} dim={dim} vdim={vdim} rank={decay_rank}")
        if not tau > 0:
            raise ValueError(f"gated linear attention: tau must be positive, got {tau}")
        self.width, self.n_heads, self.dim, self.vdim = int(width), int(n_heads), int(dim), int(vdim)
        self.tau, self.rank, self.eps = float(tau), int(decay_rank), float(eps)

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, vv, w = self.n_heads * self.dim, self.n_heads * self.vdim, self.width
        return {"q_proj": ParamSpec((qk, w)), "k_proj": ParamSpec((qk, w)), "v_proj": ParamSpec((vv, w)),
                "g_proj": ParamSpec((vv, w)), "a1_proj": ParamSpec((self.rank, w)), "a2_proj": ParamSpec((qk, self.rank)),
                "a2_proj.bias": ParamSpec((qk,)), "o_proj": ParamSpec((w, vv)), "norm": ParamSpec((self.vdim,), "norm")}

    def cache_need(self):
        return StateNeed((self.n_heads, self.dim, self.vdim), "float32")

    def load(self, tensors, runtime) -> None:
        mats = [tensors[n] for n in ("q_proj", "k_proj", "v_proj", "g_proj", "a1_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()     # one product gives q, k, v, the gate and the decay's first step
        self.w_a2, self.w_o, self.norm = tensors["a2_proj"], tensors["o_proj"], tensors["norm"]
        self.a_bias = _as_f32(tensors["a2_proj.bias"])
        if tensors["a1_proj"].shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"gated linear attention: the decay's projections do not meet "
                             f"({tensors['a1_proj'].shape[0]} against {self.w_a2.shape[1]})")
        self.rank = int(self.w_a2.shape[1])

    def forward(self, ctx, h, residual, run) -> None:
        self._run(ctx, h, residual, run, EPI_ACCUMULATE)

    def forward_store(self, ctx, h, out, run) -> None:
        self._run(ctx, h, out, run, EPI_STORE)

    def _run(self, ctx, h, target, run, epilogue) -> None:
        state = run.state
        if state is None or not run.writes_cache:
            raise RuntimeError("gated linear attention needs a state of its own for its run")
        qk, vv = self.n_heads * self.dim, self.n_heads * self.vdim
        proj = ctx.rows("gla.proj", 2 * qk + 2 * vv + self.rank)
        linear(h, self.w_in, proj, EPI_STORE)
        z = ctx.rows("gla.decay", qk)
        linear(proj[:, 2 * qk + 2 * vv:], self.w_a2, z, EPI_STORE)
        o = ctx.rows("gla.o", vv, torch.float32)
        ops.decay_scan(proj, 0, qk, proj, 2 * qk, z, 0, o, state, ctx.cu_seqlens, ctx.seq_slot, ctx.n_seqs,
                       self.n_heads, self.dim, self.vdim, 1, ops.DECAY_SIGMOID, self.a_bias, q_scale=self.dim ** -0.5,
                       inv_tau=1.0 / self.tau, few_tokens=ctx.max_seq_tokens == 1,
                       single_tokens=ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs,
                       **_chunking(ctx, self.n_heads * self.dim * self.vdim, self.n_heads * self.dim))
        y = ctx.rows("gla.y", vv)
        ops.gated_group_norm(o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.norm, self.eps, y, self.n_heads, gate_first=False)
        linear(y, self.w_o, target, epilogue)


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    graph_safe = True

    def __init__(self, width: int, inner: int, candidate: str = "positive", bias: bool = True):
        if inner < 1:
            raise ValueError(f"minGRU: bad size inner={inner}")
        if candidate not in ("positive", "identity"):
            raise ValueError(f"minGRU: the candidate is 'positive' or 'identity', got {candidate!r}")
        self.width, self.inner, self.bias = int(width), int(inner), bool(bias)
        self.cand = ops.SCAN_CAND_POSITIVE if candidate == "positive" else ops.SCAN_CAND_IDENTITY

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, w = self.inner, self.width
        specs = {"z_proj": ParamSpec((n, w)), "x_proj": ParamSpec((n, w)), "g_proj": ParamSpec((n, w)),
                 "o_proj": ParamSpec((w, n))}
        if self.bias:
            specs.update({"z_proj.bias": ParamSpec((n,)), "x_proj.bias": ParamSpec((n,))})
        return specs

    def cache_need(self):
        return StateNeed((self.inner,), "float32")

    def load(self, tensors, runtime) -> None:
        mats = [tensors[n] for n in ("z_proj", "x_proj", "g_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()      # one product gives the gate, the candidate and the output gate
        self.w_o = tensors["o_proj"]
        self.b_z = _as_f32(tensors["z_proj.bias"]) if self.bias else None
        self.b_x = _as_f32(tensors["x_proj.bias"]) if self.bias else None

    def forward(self, ctx, h, residual, run) -> None:
        self._run(ctx, h, residual, run, EPI_ACCUMULATE)

    def forward_store(self, ctx, h, out, run) -> None:
        self._run(ctx, h, out, run, EPI_STORE)

    def _run(self, ctx, h, target, run, epilogue) -> None:
        state = run.state
        if state is None or not run.writes_cache:
            raise RuntimeError("a minGRU needs a state of its own for its run")
        n = self.inner
        proj = ctx.rows("gru.proj", 3 * n)
        linear(h, self.w_in, proj, EPI_STORE)
        y = ctx.rows("gru.y", n)
        ops.gated_scan(proj, 0, n, 2 * n, n, self.b_z, self.b_x, y, state, ctx.cu_seqlens, ctx.seq_slot, ctx.n_seqs,
                       ctx.max_seq_tokens, cand=self.cand)
        linear(y, self.w_o, target, epilogue)
