"""Gated dense feed-forward: ``down(silu(gate(h)) * up(h))``, no bias
(crates/bfi-models/src/qwen3.rs:244-250; SiLU*mul crates/bfi-core/src/cpu.rs:169-180).

The gate and up matrices are stored interleaved row by row (gate_j, up_j, gate_j+1, ...), so
one matrix product yields both and its epilogue applies the activation while the pair is still in
registers; the down product adds into the residual stream.

The activation is a family with three constants: with ``g' = min(g, limit)`` and
``u' = clamp(u, -limit, limit)`` (no clamping without a limit),
``act = g' * sigmoid(gate_alpha * g') * (u' + up_shift)``.  ``gate_alpha`` 1, no limit and
``up_shift`` 0 is SiLU(gate) * up.  ``activation`` ``"gelu_tanh"`` is the other member:
``act = gelu_tanh(g) * u`` with ``gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``; the
three constants do not apply to it.

``dense_mlp`` is the feed-forward without a gate: ``W_down act(W_up h + b_up) + b_down`` with the tanh
GELU; the biases may be absent.  The kernel that applies bias and activation also writes ``b_down``
into the float32 target rows, into which the down product then accumulates.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, EPI_SWIGLU, GATE_GELU_TANH, linear
from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "silu", gate_alpha: float = 1.0,
                 limit: float = None, up_shift: float = 0.0):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp supports the silu and gelu_tanh activations, got {activation!r}")
        self.activation = activation
        if limit is not None and not limit > 0:
            raise ValueError(f"gated_mlp: the clamp limit must be positive, got {limit}")
        self.width, self.inner = int(width), int(inner)
        self.gate_alpha, self.limit, self.up_shift = float(gate_alpha), (None if limit is None else float(limit)), float(up_shift)
        self.plain_silu = activation == "silu" and self.gate_alpha == 1.0 and self.limit is None and self.up_shift == 0.0
        if activation == "gelu_tanh" and not (self.gate_alpha == 1.0 and self.limit is None and self.up_shift == 0.0):
            raise ValueError("gated_mlp: the gelu_tanh activation takes no slope, clamp or shift")
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate_proj": ParamSpec((self.inner, self.width)),
                "up_proj": ParamSpec((self.inner, self.width)),
                "down_proj": ParamSpec((self.width, self.inner))}

    def load(self, tensors, runtime) -> None:
        g, u = tensors["gate_proj"], tensors["up_proj"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inner, self.width).contiguous()
        self.w_down = tensors["down_proj"]

    def forward(self, ctx, h, residual) -> None:
        act = ctx.rows("mlp.act", self.inner)
        gate = None if self.plain_silu else (self.gate_alpha, self.limit or 0.0, self.up_shift)
        if self.activation == "gelu_tanh":
            gate = (1.0, 0.0, 0.0, GATE_GELU_TANH)
        linear(h, self.w_gate_up, act, EPI_SWIGLU, gate)
        linear(act, self.w_down, residual, EPI_ACCUMULATE)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "gelu_tanh", bias: bool = True):
        if activation != "gelu_tanh":
            raise ValueError(f"dense_mlp supports the gelu_tanh activation, got {activation!r}")
        self.width, self.inner, self.bias = int(width), int(inner), bool(bias)
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"up_proj": ParamSpec((self.inner, self.width)), "down_proj": ParamSpec((self.width, self.inner))}
        if self.bias:
            specs.update({"up_proj.bias": ParamSpec((self.inner,)), "down_proj.bias": ParamSpec((self.width,))})
        return specs

    def load(self, tensors, runtime) -> None:
        self.w_up, self.w_down = tensors["up_proj"], tensors["down_proj"]
        if self.bias:
            self.b_up, self.b_down = tensors["up_proj.bias"].contiguous(), tensors["down_proj.bias"].contiguous()

    def forward_store(self, ctx, h, out) -> None:
        act = ctx.rows("mlp.act", self.inner)
        linear(h, self.w_up, act, EPI_STORE)
        if self.bias:
            ops.bias_act(act, self.b_up, act, fill=out, fill_bias=self.b_down)
            linear(act, self.w_down, out, EPI_ACCUMULATE)
        else:
            ops.bias_act(act, None, act)
            linear(act, self.w_down, out, EPI_STORE)

    def forward(self, ctx, h, residual) -> None:
        y = ctx.rows("mlp.out", self.width, torch.float32)
        self.forward_store(ctx, h, y)
        ops.residual_add(residual, y)
