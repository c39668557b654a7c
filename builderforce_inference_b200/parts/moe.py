"""A routed feed-forward (mixture of experts), with an optional expert that every token uses.

Router: ``z = W_router h`` in float32 (h as the activation dtype holds it), ``s = softmax(z)`` over
all experts.  Experts are chosen by ``s + correction`` (a stored vector): they form
``n_groups`` equal groups of neighbours, a group counts by its best choice score, only experts of
the ``keep_groups`` best groups can be chosen, and of those the ``top`` best are.  The chosen
experts' weights are their ``s`` (not renormalised) times ``weight_scale``.  An expert is
``W_down (silu(W_gate h) * (W_up h))``; the output is the weighted sum of the chosen experts'.
The shared expert has the same form (its own inner size) and is added multiplied by
``sigmoid(W_sg h)``, one number per token.

The router's matrix and the shared expert's gate row are kept as one float32 matrix; one kernel
makes the logits and the gate's input from it in float32 and decides (``kernels/ops.moe_router``).  The experts' weights are kept
as two matrices for all experts (gate and up rows interleaved, expert after expert; the down
matrices side by side), which serve two ways of computing: a step with few (token, expert) pairs
reads only the chosen experts' weights (``kernels/ops.moe_gate_up``, ``moe_down``); a bfloat16 step
with at least ``DENSE_PAIRS_PER_EXPERT`` pairs per expert, which touches nearly every expert anyway,
runs the two dense products over all experts on the tensor cores and multiplies the activations by
the chosen experts' weights, 0 for the others, in between (``moe_weigh_dense``); the shared expert
stands behind the routed ones in both matrices and is weighed by its gate there, so the dense way is
two products and one kernel between them.  In the other way the shared expert runs through dense
products of its own.  Nothing here reads a choice back to the host, so a step through
this part can be captured in a graph.

Variants, each a parameter: ``score`` ``"sigmoid"`` (``s = sigmoid(z)``, every expert by itself, instead
of the softmax); ``group_top`` (a group counts by the sum of its ``group_top`` best choice scores
instead of the best one); ``correction`` false (no stored vector: experts are chosen by ``s``);
``expert`` ``"relu_squared"`` (an expert is ``W_down relu(W_up h)^2``, without a gate matrix: the up
matrices of all experts are one matrix, and in the dense way the activation is applied by the
kernel that weighs); ``shared_gate`` false (the shared expert is added as it is).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, EPI_SWIGLU, linear
from .base import FEED_FORWARDS, FeedForward, ParamSpec


DENSE_PAIRS_PER_EXPERT = 2      # from this many (token, expert) pairs per expert on, every expert is computed for every token


@FEED_FORWARDS.register("mixture_of_experts")
class RoutedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, n_experts: int, top: int, inner: int, n_groups: int = 1, keep_groups: int = 1,
                 shared_inner: Optional[int] = None, correction: bool = True, weight_scale: float = 1.0,
                 score: str = "softmax", group_top: int = 1, expert: str = "gated_silu", shared_gate: bool = True):
        if n_experts < 1 or not 1 <= top <= n_experts or inner < 1:
            raise ValueError(f"routed feed-forward: bad sizes experts={n_experts} top={top} inner={inner}")
        if n_groups < 1 or n_experts % n_groups != 0 or not 1 <= keep_groups <= n_groups:
            raise ValueError(f"routed feed-forward: {n_experts} experts in {n_groups} groups, {keep_groups} kept")
        if keep_groups * (n_experts // n_groups) < top:
            raise ValueError(f"routed feed-forward: {keep_groups} groups of {n_experts // n_groups} experts cannot give {top}")
        self.width, self.n_experts, self.top, self.inner = int(width), int(n_experts), int(top), int(inner)
        self.n_groups, self.keep_groups = int(n_groups), int(keep_groups)
        self.shared_inner = None if shared_inner is None else int(shared_inner)
        self.has_correction, self.weight_scale = bool(correction), float(weight_scale)
        if score not in ("softmax", "sigmoid") or expert not in ("gated_silu", "relu_squared") or group_top < 1:
            raise ValueError(f"routed feed-forward: score {score!r}, expert {expert!r}, group_top {group_top}")
        self.score = ops.SCORE_SIGMOID if score == "sigmoid" else ops.SCORE_SOFTMAX
        self.group_top = int(group_top)
        self.gated = expert == "gated_silu"
        self.kind = ops.EXPERT_GATED_SILU if self.gated else ops.EXPERT_RELU_SQUARED
        self.shared_gate = bool(shared_gate) and self.shared_inner is not None

    def param_specs(self) -> Dict[str, ParamSpec]:
        w = self.width
        specs = {"router": ParamSpec((self.n_experts, w))}
        if self.has_correction:
            specs["correction"] = ParamSpec((self.n_experts,))
        for e in range(self.n_experts):
            if self.gated:
                specs[f"experts.{e}.gate_proj"] = ParamSpec((self.inner, w))
            specs[f"experts.{e}.up_proj"] = ParamSpec((self.inner, w))
            specs[f"experts.{e}.down_proj"] = ParamSpec((w, self.inner))
        if self.shared_inner is not None:
            if self.gated:
                specs["shared.gate_proj"] = ParamSpec((self.shared_inner, w))
            specs["shared.up_proj"] = ParamSpec((self.shared_inner, w))
            specs["shared.down_proj"] = ParamSpec((w, self.shared_inner))
            if self.shared_gate:
                specs["shared.gate"] = ParamSpec((1, w))
        return specs

    def load(self, tensors, runtime) -> None:
        kinds = ("gate_proj", "up_proj", "down_proj") if self.gated else ("up_proj", "down_proj")
        per = len(kinds)
        mats = [tensors[f"experts.{e}.{kind}"] for e in range(self.n_experts) for kind in kinds]
        if self.shared_inner is not None:
            mats += [tensors[f"shared.{kind}"] for kind in kinds]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        n_all = self.n_experts + (1 if self.shared_inner is not None else 0)
        # gate and up rows interleaved, or the up rows alone; the shared expert stands behind the routed
        # ones in both matrices, so the dense way is two products for all of them; the other way reads
        # it through views (and its own down matrix)
        if self.gated:
            gu = [torch.stack([mats[per * e], mats[per * e + 1]], dim=1).reshape(-1, self.width) for e in range(n_all)]
        else:
            gu = [mats[per * e] for e in range(n_all)]
        downs = [mats[per * e + per - 1] for e in range(n_all)]
        rows = [tensors["router"].float()]
        if self.shared_gate:
            rows.append(tensors["shared.gate"].float())
        if self.shared_inner is not None:
            self.ws_down = downs[-1].contiguous()
        self.w_gu_all = torch.cat(gu, dim=0).contiguous()                  # [(E * ff + shared) * (2 | 1), width]
        self.w_down_all = torch.cat(downs, dim=1).contiguous()             # [width, E * ff + shared]
        routed = self.n_experts * self.inner
        rows_per = 2 if self.gated else 1
        self.w_gu = self.w_gu_all[:rows_per * routed]                      # [E * (2 | 1) * ff, width]
        self.w_down = self.w_down_all[:, :routed]                          # [width, E * ff], rows of the wider matrix
        self.routed_rows = rows_per * routed                               # the shared expert's rows follow
        self.w_router = torch.cat(rows, dim=0).contiguous()                # float32: the logits are float32 sums
        self.correction = tensors["correction"].float().contiguous() if self.has_correction else None

    def forward_store(self, ctx, h, out) -> None:
        self._run(ctx, h, out, accumulate=False)

    def forward(self, ctx, h, residual) -> None:
        self._run(ctx, h, residual, accumulate=True)

    def _run(self, ctx, h, target, accumulate: bool) -> None:
        n = h.shape[0]
        shared = self.shared_inner is not None
        idx = ctx.rows("moe.idx", self.top, torch.int32)
        wts = ctx.rows("moe.weight", self.top, torch.float32)
        gate = ctx.rows("moe.gate", 1, torch.float32).view(-1) if self.shared_gate else None
        ops.moe_router(h, self.w_router, self.n_experts, self.correction, ctx.token_slot, idx, wts, self.top, self.n_groups,
                       self.keep_groups, self.weight_scale, gate, self.score, self.group_top)
        if h.dtype == torch.bfloat16 and self.w_gu_all.dtype == torch.bfloat16 \
                and n * self.top >= DENSE_PAIRS_PER_EXPERT * self.n_experts:
            tail = self.shared_inner or 0
            act = ctx.rows("moe.act.dense", self.n_experts * self.inner + tail)
            linear(h, self.w_gu_all, act, EPI_SWIGLU if self.gated else EPI_STORE)
            ops.moe_weigh_dense(act, self.n_experts, idx, wts, ctx.token_slot, tail, gate, self.kind)
            linear(act, self.w_down_all, target, EPI_ACCUMULATE if accumulate else EPI_STORE)
            return
        ys = None
        if shared:
            act_s = ctx.rows("moe.shared.act", self.shared_inner)
            if self.gated:
                linear(h, self.w_gu_all[self.routed_rows:], act_s, EPI_SWIGLU)
            else:       # the up product with its activation: the chosen-experts kernel, for one expert all use
                ops.moe_gate_up(h, self.w_gu_all[self.routed_rows:], 1, None, ctx.token_slot, act_s, self.kind)
            ys = ctx.rows("moe.shared.out", self.width, torch.float32)
            linear(act_s, self.ws_down, ys, EPI_STORE)
        act = ctx.rows("moe.act", self.top * self.inner).view(n * self.top, self.inner)
        ops.moe_gate_up(h, self.w_gu, self.n_experts, idx, ctx.token_slot, act, self.kind)
        ops.moe_down(act, self.w_down, self.n_experts, idx, wts, ctx.token_slot, target, ys, gate, accumulate)
