"""Norms.  RMSNorm, fused with the residual add that precedes it; LayerNorm with weight and bias, fused with the
scaled and gated residual sum of a post-norm layer.

``y = x * rsqrt(mean(x^2) + eps) * w``: normalise first, multiply by the weight second, no ``1 + w``
and no bias (src/iian/graph.cpp:105-114).  The sum of squares and the residual sum are float32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, NormedAddend, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``; optional ``weight_offset`` (default 0): the stored weight ``w`` is used as
    ``weight_offset + w`` (a weight kept around zero has ``weight_offset`` 1).

    ``delta`` may be a pair of tensors (the outputs of two sub-layers that read the same norm): the stream becomes
    ``x + (d1 + d2)``, summed in float32; or a ``NormedAddend`` (a sub-layer output that passes a norm of its own on its way
    into the stream): both norms and the sum are one kernel.  ``as_addend(y)`` wraps a sub-layer output for THIS norm to be
    applied to it on its way into the stream."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.offset = float(spec.params.get("weight_offset", 0.0))
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="zeros_jitter" if self.offset else "ones_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors["weight"].to(torch.float32)                            # exact widening; the kernel multiplies in float32
        self.weight = (w + self.offset if self.offset else w).contiguous()

    def kernel_libraries(self):
        return ("elementwise", "residual_ops")

    def foldable(self):
        return (self.weight, self.eps) if self.weight is not None else None

    def as_addend(self, y: torch.Tensor) -> NormedAddend:
        return NormedAddend(y, self.weight, self.eps)

    def forward(self, residual: torch.Tensor, delta, ctx, delta_scale: float = 1.0) -> torch.Tensor:
        """``delta_scale``: the stream becomes ``x + delta_scale * delta`` (a design that adds its sub-layers' outputs with a
        factor)."""
        out = ctx.buf("normed", residual.shape, self.dtype)
        if isinstance(delta, NormedAddend):
            if delta_scale != 1.0:
                raise ValueError("rms_norm: a normalised addend takes no factor")
            ops.kernels().normed_add_rms_norm(residual, delta.y, delta.weight, delta.eps, delta.extra, self.weight, self.eps, out)
            return out
        if delta_scale != 1.0 and delta is not None:
            if isinstance(delta, tuple):
                raise ValueError("rms_norm: a pair of addends takes no factor")
            ops.kernels().scaled_add_rms_norm(residual, delta, delta_scale, self.weight, self.eps, out)
            return out
        if isinstance(delta, tuple):
            live = [d for d in delta if d is not None]
            if len(live) == 2:
                ops.kernels().add2_rms_norm(residual, live[0], live[1], self.weight, self.eps, out)
                return out
            delta = live[0] if live else None
        ops.kernels().add_rms_norm(residual, delta, self.weight, self.eps, out)
        return out


@register_norm("layer_norm")
class LayerNorm(Norm):
    """params: ``size``, ``eps``.  ``y = (x - mean) / sqrt(var + eps) * w + b`` with ``var`` the mean of the squared
    deviations; sums in float32.

    Two uses.  As the norm that closes a model (``forward``): the stream is normalised into the activation dtype.  As the
    norm AFTER a sub-layer's sum in a post-norm layer (``sum_norm``): ``LayerNorm(alpha * x + sub * sigmoid(gate))``,
    the scaled skip, the gated sub-layer output and the norm in one kernel, leaving the new float32 stream and its copy in
    the activation dtype for the products that read it next."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_jitter"), "bias": TensorSpec((self.size,))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("postnorm",)

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx) -> torch.Tensor:
        out = ctx.buf("normed", residual.shape, self.dtype)
        ops.kernels().gated_add_layer_norm(residual, delta, None, None, self.weight, self.bias, 1.0, self.eps, None, out)
        return out

    def sum_norm(self, x: torch.Tensor, alpha: float, sub: torch.Tensor, gate: Optional[torch.Tensor],
                 gate_bias: Optional[torch.Tensor], ctx, name: str, want_act: bool = True):
        """``(stream float32, the same in the activation dtype)`` of ``LayerNorm(alpha * x + sub * sigmoid(gate + gate_bias))``.
        In the 32-bit path the two are one tensor; without ``want_act`` the second is None."""
        out = ctx.buf(f"stream_{name}", x.shape, torch.float32)
        if self.dtype == torch.float32:
            ops.kernels().gated_add_layer_norm(x, sub, gate, gate_bias, self.weight, self.bias, alpha, self.eps, out, None)
            return out, out
        if not want_act:
            ops.kernels().gated_add_layer_norm(x, sub, gate, gate_bias, self.weight, self.bias, alpha, self.eps, out, None)
            return out, None
        act = ctx.buf(f"stream_act_{name}", x.shape, self.dtype)
        ops.kernels().gated_add_layer_norm(x, sub, gate, gate_bias, self.weight, self.bias, alpha, self.eps, out, act)
        return out, act
