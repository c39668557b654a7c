"""``out = a @ w.T`` with a choice of epilogue: the one place that decides which matrix-product
kernel runs for a shape and a pair of storage types.

* float32 anywhere in the product: the CUDA-core kernels (float32 multiply-add; this is the
  whole of the 32-bit path, no tensor-core mode is involved);
* bfloat16 x bfloat16: few rows stream the weights once through the tensor-core skinny kernel,
  many rows run the tcgen05 kernel; shapes those kernels refuse go to the CUDA-core kernels.
"""
from __future__ import annotations

import torch

from . import ops
from .ops import EPI_ACCUMULATE, EPI_STORE, EPI_SWIGLU  # noqa: F401  (re-exported)

_fast = None


def _fast_ops():
    global _fast
    if _fast is None:
        from . import fast_ops
        _fast = fast_ops
    return _fast


GATE_SIGMOID, GATE_GELU_TANH = 0, 1      # kinds of the gated epilogue's activation


def _set_gate(fast: bool, alpha: float, limit: float, shift: float, kind: int = GATE_SIGMOID) -> None:
    from ctypes import c_float, c_int

    from .library import library
    for name in (("core", "fast") if fast else ("core",)):
        library(name).lib.bfi_set_gate_kind(c_int(kind), c_float(alpha), c_float(limit), c_float(shift))


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE, gate=None) -> None:
    """``gate``: with the gated epilogue, the activation's constants ``(alpha, limit, shift)``:
    ``g' * sigmoid(alpha * g') * (u' + shift)`` with gate and up clamped at ``limit`` (0: not
    clamped); None is SiLU(gate) * up.  A fourth value names the activation's kind:
    ``GATE_GELU_TANH`` is ``gelu_tanh(g) * u`` (the three constants are then unused).  The kernels
    take them along as launch arguments."""
    fast = a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if gate is not None and epilogue == EPI_SWIGLU:
        _set_gate(fast, *gate)
        try:
            linear(a, w, out, epilogue)
        finally:
            _set_gate(fast, 1.0, 0.0, 0.0)
        return
    if fast:
        if _fast_ops().linear_bf16(a, w, out, epilogue):
            return
    ops.gemm_simt(a, w, out, epilogue)
