"""RMS norm: ``y = x * rsqrt(mean(x^2) + eps) * w`` over the last dim, the weight as stored
(crates/bfi-core/src/cpu.rs:92-122), or, with ``offset``, ``offset + w`` (a weight stored around zero
enters as ``1 + w``; the sum is made once at load, in float32).  The statistics are float32; the
input is the float32 residual stream and the output is in the activation dtype.  ``add_to`` is the
same norm applied to a sublayer's float32 output on its way into the residual stream."""
from __future__ import annotations

from typing import Dict

from ..kernels import ops
from .base import NORMS, Norm, ParamSpec


@NORMS.register("rms")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, offset: float = 0.0):
        self.width = int(width)
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "norm")}

    def load(self, tensors, runtime) -> None:
        self.weight = tensors["weight"]
        if self.offset != 0.0:
            self.weight = (self.weight.float() + self.offset).contiguous()

    def forward(self, ctx, x, rows=None, tag: str = "norm.out"):
        n = x.shape[0] if rows is None else rows.numel()
        out = ctx.rows(tag, self.width, n_rows=n)
        ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

    def add_to(self, ctx, residual, y, then=None, mult: float = 1.0, gate=None, gate_bias=None, conv=None):
        """``residual += mult * norm(y)``: both float32 ``[tokens, width]``.  With ``gate`` (logits of
        the stream's shape, and an optional bias) ``y`` is first multiplied by ``sigmoid(gate + bias)``.
        With ``then`` (the norm that reads the residual stream next) its output is made in the same
        kernel and returned.  ``conv``: see ``ops.norm_add``."""
        if not isinstance(then, RMSNorm):
            ops.norm_add(residual, y, self.weight, self.eps, mult=mult, gate=gate, gate_bias=gate_bias, conv=conv)
            return None if then is None else then.forward(ctx, residual)
        out = ctx.rows("norm.out", then.width)
        ops.norm_add(residual, y, self.weight, self.eps, next_w=then.weight, next_eps=then.eps, out=out, mult=mult,
                     gate=gate, gate_bias=gate_bias)
        return out
