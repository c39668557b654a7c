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
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels.linear import EPI_ACCUMULATE, EPI_SWIGLU, GATE_GELU_TANH, linear
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
