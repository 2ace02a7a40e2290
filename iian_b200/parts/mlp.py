"""Dense gated feed-forward: ``y = Wdown (act(Wgate h) * (Wup h))``, parallel gate, no biases
(src/iian/graph.cpp:116-163 with ``FfnOp::SILU`` / ``FfnGate::PAR``, src/iian/arch/qwen3.cpp:97).
``silu(z) = z / (1 + exp(-z))`` (third_party/ggml/src/ggml-cpu/vec.h:1046-1048).

Gate and up projections run as one matrix product over the rows of both, stacked at load time in groups of
8 (8 gate rows, then the 8 up rows of the same features, ...), so that a product kernel that owns 16
consecutive rows holds both halves of 8 features and can apply SiLU(gate) * up in its epilogue.  If the
intermediate size is no multiple of 8 the rows are stacked as ``Wgate | Wup``.

``activation``: ``silu`` or ``gelu_tanh`` (``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``); the second has no
fused product epilogue and runs as product, then activation kernel.  ``stack_rows`` puts further rows that read the same
input (a gate of the residual) under ``Wgate | Wup`` so that one product serves all.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, Prenormed, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (``silu`` | ``gelu_tanh``); optional ``names``: the
    local tensor names of (gate, up, down)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.params.get("activation", "silu")
        if act not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp: activation '{act}' has no kernel (silu, gelu_tanh)")
        self.activation = act
        self.names = tuple(spec.params.get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.w_gate_up = self.w_down = None
        self.interleave = 0
        self.extra_rows = None
        self.w_all = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {
            self.names[0]: TensorSpec((self.inter, self.hidden)),
            self.names[1]: TensorSpec((self.inter, self.hidden)),
            self.names[2]: TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        if self.inter % 8 == 0:
            k = g.shape[1]
            self.w_gate_up = torch.stack([g.view(self.inter // 8, 8, k), u.view(self.inter // 8, 8, k)], dim=1) \
                .reshape(2 * self.inter, k).contiguous()
            self.interleave = 8
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
            self.interleave = 0
        self.w_down = tensors[self.names[2]].contiguous()

    def stack_rows(self, rows: torch.Tensor) -> None:
        """Further rows [m, hidden] to be multiplied with the input in the same product as gate and up (call after
        ``bind``); ``forward(..., with_extra=True)`` returns their columns beside the output."""
        self.extra_rows = rows
        ws = [self.w_gate_up, rows]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.to(torch.float32) for w in ws]
        self.w_all = torch.cat(ws, dim=0).contiguous()

    def kernel_libraries(self):
        return ("elementwise", "gemm_simt") + (("postnorm",) if self.activation != "silu" else ())

    folds_norm_out = True

    def takes_prenormed(self, n_rows: int) -> bool:
        k = ops.kernels()
        return (hasattr(k, "can_take_prenormed") and self.interleave == 8 and self.activation == "silu"
                and k.can_take_prenormed(n_rows, self.w_gate_up, self.dtype))

    def _forward_general(self, x, ctx, with_extra: bool):
        """Product over gate, up and any stacked rows, then the activation kernel (any activation)."""
        k = ops.kernels()
        n = x.shape[0]
        w = self.w_all if self.extra_rows is not None else self.w_gate_up
        wide = ctx.buf("gate_up", (n, w.shape[0]), self.dtype)
        k.linear(x, w, wide)
        act = ctx.buf("ffn_act", (n, self.inter), self.dtype)
        k.gated_act(wide[:, : 2 * self.inter], act, self.interleave, self.activation)
        out = ctx.buf("ffn_out", (n, self.hidden), self.dtype)
        k.linear(act, self.w_down, out)
        if with_extra:
            return out, (wide[:, 2 * self.inter:] if self.extra_rows is not None else None)
        return out

    def forward(self, x, ctx, norm_out=None, with_extra: bool = False):
        if with_extra or self.activation != "silu":
            return self._forward_general(x, ctx, with_extra)
        k = ops.kernels()
        scale = None
        if isinstance(x, Prenormed):
            x, scale = x.x, x.scale
        n = x.shape[0]
        act = ctx.buf("ffn_act", (n, self.inter), self.dtype)
        if scale is not None:
            k.linear_swiglu(x, self.w_gate_up, act, row_scale=scale)
        elif hasattr(k, "can_fuse_swiglu") and k.can_fuse_swiglu(x, self.w_gate_up, self.interleave):
            k.linear_swiglu(x, self.w_gate_up, act)            # the activation rides in the product's epilogue
        else:
            gate_up = ctx.buf("gate_up", (n, 2 * self.inter), self.dtype)
            k.linear(x, self.w_gate_up, gate_up)
            k.swiglu(gate_up, act, self.interleave)
        if norm_out is not None and hasattr(k, "can_fuse_norm") and k.can_fuse_norm(act, self.w_down):
            return norm_out.take(k, act, self.w_down, ctx)
        out = ctx.buf("ffn_out", (n, self.hidden), self.dtype)
        k.linear(act, self.w_down, out)
        return out


@register_feed_forward("plain_mlp")
class PlainMLP(FeedForward):
    """A feed-forward without a gate: ``y = Wdown act(Wup h)``.

    params: ``hidden_size``, ``intermediate_size``, ``activation``: ``xielu`` (two learned numbers p, q in a tensor of
    their own: ``z > 0: softplus(p) z^2 + z / 2``, else ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``); optional
    ``names``: the local tensor names of (up, down, the activation's numbers)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.params.get("activation", "xielu")
        if act != "xielu":
            raise ValueError(f"plain_mlp: activation '{act}' has no kernel (xielu)")
        self.activation = act
        self.names = tuple(spec.params.get("names", ("up", "down", "act")))
        self.w_up = self.w_down = self.act_numbers = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.names[0]: TensorSpec((self.inter, self.hidden)), self.names[1]: TensorSpec((self.hidden, self.inter)),
                self.names[2]: TensorSpec((2,), init="zeros_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.names[0]].contiguous()
        self.w_down = tensors[self.names[1]].contiguous()
        self.act_numbers = tensors[self.names[2]].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("residual_ops", "gemm_simt")

    def forward(self, x, ctx):
        k = ops.kernels()
        n = x.shape[0]
        up = ctx.buf("ffn_up", (n, self.inter), self.dtype)
        k.linear(x, self.w_up, up)
        act = ctx.buf("ffn_act", (n, self.inter), self.dtype)
        k.xielu(up, self.act_numbers, act)
        out = ctx.buf("ffn_out", (n, self.hidden), self.dtype)
        k.linear(act, self.w_down, out)
        return out
