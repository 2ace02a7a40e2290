"""Routed experts: a feed-forward made of many small gated feed-forwards, of which each token uses a few.

``z = Wrouter h`` in float32; scores ``s = sigmoid(z)``; a token takes the ``top`` experts with the largest scores and
weighs them by those scores as they are (no renormalisation).  With ``weight_on = "input"`` the weight multiplies what
the expert reads: ``y = sum_e expert_e(s_e h)``, ``expert(u) = Wdown (act(Wgate u) * (Wup u))``, no biases.

The step never learns on the host how many rows an expert got.  A routing kernel picks experts, a one-block plan
kernel sorts the (token, choice) rows by expert and lists the row tiles, the rows are gathered (and scaled), two
grouped products run over the sorted rows -- gate and up with the activation in the epilogue, then down -- and a last
kernel adds a token's expert outputs in the order of its choices.  All sizes are fixed by the number of tokens, so the
part can be recorded into a CUDA graph.

Two further forms, chosen by parameters.  ``score = "table"``: there is no router; row ``token id`` of an integer table
[vocab, top] names the token's experts (the entries of a row differ) and every one weighs ``1 / top``.  ``weight_on =
"output"``: the weight multiplies what the expert returns, ``y = sum_e w_e expert_e(h)``.  ``activation =
"clamped_swish"``: ``g = min(Wgate u, limit)``, ``v = clamp(Wup u, -limit, limit)``, the expert's hidden row is
``g sigmoid(1.702 g) (v + 1)``.

``score = "softmax_top"``: the router has a bias (``router.b``, float32 sum), the ``top`` experts with the largest biased
logits are taken and weighed by the softmax over those logits ALONE.  ``shared_intermediate_size``: one more gated
feed-forward of that width (tensors ``shared.gate / up / down``, same activation) that every token uses; its output is added
to the experts' sum in the kernel that forms it.

``stack_rows`` puts further rows that read the same input (a gate of the residual) under the router's, so that one
product with float32 output serves both.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``hidden_size``, ``num_experts``, ``top``, ``intermediate_size`` (of one expert), ``activation``
    (``silu`` | ``gelu_tanh`` | ``clamped_swish`` with ``limit``), ``score`` (``sigmoid`` | ``table`` with ``vocab_size``),
    ``weight_on`` (``input`` | ``output``)."""

    SWISH_ALPHA = 1.702         # fixed by the clamped activation (also in the kernels)

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.experts = int(p["num_experts"])
        self.top = int(p["top"])
        self.inter = int(p["intermediate_size"])
        self.activation = p.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh", "clamped_swish"):
            raise ValueError(f"routed_experts: activation '{self.activation}' has no kernel")
        self.limit = float(p.get("limit", 0.0))
        if self.activation == "clamped_swish" and self.limit <= 0:
            raise ValueError("routed_experts: the clamped activation needs a positive limit")
        self.score = p.get("score", "sigmoid")
        self.weight_on = p.get("weight_on", "input")
        if self.score not in ("sigmoid", "softmax_top", "table") or self.weight_on not in ("input", "output"):
            raise ValueError("routed_experts: score is 'sigmoid', 'softmax_top' or 'table', weight_on 'input' or 'output'")
        self.shared_inter = int(p.get("shared_intermediate_size", 0) or 0)
        self.shared = None
        if self.shared_inter:
            if self.activation not in ("silu", "gelu_tanh"):
                raise ValueError("routed_experts: the shared expert takes silu or gelu_tanh")
            from ..config.spec import PartSpec
            from .mlp import GatedMLP
            self.shared = GatedMLP(PartSpec("gated_mlp", {"hidden_size": self.hidden, "intermediate_size": self.shared_inter,
                                                          "activation": self.activation,
                                                          "names": ("shared.gate", "shared.up", "shared.down")}), dtype, device)
        self.router_bias = None
        self.vocab = int(p["vocab_size"]) if self.score == "table" else 0
        self.needs_tokens = self.score == "table"       # forward wants to know which token each row belongs to
        if not 0 < self.top <= self.experts:
            raise ValueError(f"routed_experts: top {self.top} of {self.experts} experts")
        self.w_router = self.w_gate = self.w_up = self.w_down = self.w_gate_up = None
        self.extra_rows = None
        self.table = None

    def tensors(self) -> Dict[str, TensorSpec]:
        if self.score == "table":
            t = {"table": TensorSpec((self.vocab, self.top), kind="int", init=f"distinct_rows:{self.experts}")}
        else:
            t = {"router": TensorSpec((self.experts, self.hidden))}
            if self.score == "softmax_top":
                t["router.b"] = TensorSpec((self.experts,))
        if self.shared is not None:
            t.update(self.shared.tensors())
        for e in range(self.experts):
            t[f"e{e}.gate"] = TensorSpec((self.inter, self.hidden))
            t[f"e{e}.up"] = TensorSpec((self.inter, self.hidden))
            t[f"e{e}.down"] = TensorSpec((self.hidden, self.inter))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.score == "table":
            self.table = tensors["table"].to(torch.int32).contiguous()
        else:
            self._router = tensors["router"]
            self.w_router = self._router.contiguous()
            if self.score == "softmax_top":
                self.router_bias = tensors["router.b"].to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared.bind({k: t for k, t in tensors.items() if k.startswith("shared.")})
        gate = torch.stack([tensors[f"e{e}.gate"] for e in range(self.experts)])
        up = torch.stack([tensors[f"e{e}.up"] for e in range(self.experts)])
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        if self.inter % 8 == 0:
            # gate and up rows interleaved in groups of 8, the layout a product kernel wants for act(gate) * up in its epilogue
            E, F, W = self.experts, self.inter, self.hidden
            self.w_gate_up = torch.stack([gate.view(E, F // 8, 8, W), up.view(E, F // 8, 8, W)], dim=2).reshape(E, 2 * F, W).contiguous()
            self.w_gate = self.w_up = None
        else:
            self.w_gate_up, self.w_gate, self.w_up = None, gate.contiguous(), up.contiguous()

    def stack_rows(self, rows: torch.Tensor) -> None:
        if self.score == "table":
            raise ValueError("routed_experts: without a router there is no product to carry further rows")
        self.extra_rows = rows
        ws = [self._router, rows]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.to(torch.float32) for w in ws]
        self.w_router = torch.cat(ws, dim=0).contiguous()

    def kernel_libraries(self):
        if self.shared is not None:
            return tuple(set(("moe", "gemm_simt") + tuple(self.shared.kernel_libraries())))
        if self.activation == "clamped_swish" and self.dtype == torch.bfloat16:
            return ("moe", "gemm_simt", "postnorm")      # the activation between the two tcgen05 products
        return ("moe", "gemm_simt")        # in bfloat16 the products' fast forms come with gemm_simt (the grouped tcgen05 one too)

    def forward(self, x, ctx, with_extra: bool = False, rows=None):
        """``rows`` (int32, optional): the step's token each row of ``x`` belongs to, when ``x`` holds selected rows only
        (a part with ``needs_tokens`` is told; without it row r is token r)."""
        k = ops.kernels()
        n = x.shape[0]
        top, E = self.top, self.experts
        m = n * top
        if n == 0:
            out = ctx.buf("ffn_out", (0, self.hidden), self.dtype)
            return (out, None) if with_extra else out
        ids = ctx.buf("expert_ids", (n, top), torch.int32)
        wts = ctx.buf("expert_weights", (n, top), torch.float32)
        logits = None
        if self.score == "table":
            k.moe_table_route(ctx.tokens, rows, self.table, E, ids, wts, 1.0 / top)
        else:
            logits = ctx.buf("router_logits", (n, self.w_router.shape[0]), torch.float32)
            k.linear(x, self.w_router, logits)
            if self.score == "softmax_top":
                k.moe_route_softmax(logits[:, :E], self.router_bias, top, ids, wts)
            else:
                k.moe_route(logits[:, :E], top, ids, wts)
        on_input = self.weight_on == "input"
        on_tc = (self.w_gate_up is not None and hasattr(k, "moe_tcgen05_ok")
                 and k.moe_tcgen05_ok(self.dtype, self.hidden, self.inter, self.activation))
        tile_rows = k.MOE_TC_TILE_ROWS if on_tc else k.moe_tile_rows()
        max_tiles = k.moe_max_tiles(m, E, tile_rows)
        offsets = ctx.buf("expert_offsets", (E + 1,), torch.int32)
        pos = ctx.buf("expert_pos", (m,), torch.int32)
        tiles = ctx.buf("expert_tiles", (1 + 2 * max_tiles,), torch.int32)
        k.moe_plan(ids, E, offsets, pos, tiles, tile_rows)
        xs = ctx.buf("expert_in", (m, self.hidden), self.dtype)
        k.moe_scatter(x, pos, wts if on_input else None, xs, top)
        act = ctx.buf("expert_act", (m, self.inter), self.dtype)
        ys = ctx.buf("expert_out", (m, self.hidden), self.dtype)
        if on_tc and self.activation != "silu":
            wide = ctx.buf("expert_gate_up", (m, 2 * self.inter), self.dtype)
            k.moe_grouped_gemm_tc(xs, self.w_gate_up, wide, offsets, tiles, gated=False)
            k.gated_act(wide, act, 8, self.activation, self.limit)
            k.moe_grouped_gemm_tc(act, self.w_down, ys, offsets, tiles, gated=False)
        elif on_tc:
            k.moe_grouped_gemm_tc(xs, self.w_gate_up, act, offsets, tiles, gated=True)
            k.moe_grouped_gemm_tc(act, self.w_down, ys, offsets, tiles, gated=False)
        else:
            if self.w_gate_up is not None:
                k.moe_grouped_gemm(xs, self.w_gate_up, self.w_gate_up, act, offsets, tiles, self.activation, self.limit)
            else:
                k.moe_grouped_gemm(xs, self.w_gate, self.w_up, act, offsets, tiles, self.activation, self.limit)
            k.moe_grouped_gemm(act, self.w_down, None, ys, offsets, tiles)
        if self.shared is not None:
            out = self.shared.forward(x, ctx)                      # lands in "ffn_out"; the experts' sum is added onto it
            k.moe_combine_add(ys, pos, out, top, None if on_input else wts, out)
        else:
            out = ctx.buf("ffn_out", (n, self.hidden), self.dtype)
            if on_input:
                k.moe_combine(ys, pos, out, top)
            else:
                k.moe_combine(ys, pos, out, top, wts)
        if with_extra:
            return out, (logits[:, E:] if self.extra_rows is not None else None)
        return out
