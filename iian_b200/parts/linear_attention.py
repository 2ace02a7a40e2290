"""Linear attention with a decay: a recurrent mixer whose state is a matrix per head.

``q``, ``k`` (heads x dim) and ``v`` (heads x v_dim) are projections of the input, optionally through silu
(``activation``); q takes the factor ``q_scale``.  Per head

    S_t = diag(a_t) S_{t-1} + k_t v_t^T,        o_t = S_t^T q_t,        S_0 = 0

with the decay ``a_t`` acting on the rows of S (the key channels).  ``decay = "head"``: one constant per head, given in the
parameters, the same for every channel and token.  ``decay = "channel"``: a learned number per key channel and token,
``a_t = sigmoid(W2 (W1 h_t) + b)^(1 / tau)`` through a low-rank pair of matrices.

The read-out passes an RMS norm -- ``norm = "all"``: over all heads together with a weight per column;
``norm = "head"``: every head over its own v_dim entries with ONE weight vector [v_dim] shared by the heads -- is multiplied
by ``gate_act(Wg h)`` (``sigmoid`` | ``silu``), and projected by ``Wo``.

The state (float32, stored column by column in blocks of 16 columns: [heads, blocks, 16, dim rounded up to 4]) lives in the request's state slot and is carried
from step to step; a step walks the tokens it brings in order.  ``Wq | Wk | Wv | Wg`` are one product in the activation dtype (``input_rows``); the decay's first matrix is a small
product of its own, its second one a product with float32 output; decays, the state and the recurrence are float32 in both
dtypes (``csrc/decay_scan.cu``).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer


@register_mixer("decay_linear_attention")
class DecayLinearAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``dim``, ``v_dim``, ``activation`` (None | ``silu``), ``q_scale``, ``decay``
    (``head`` with ``head_decay``: a number per head | ``channel`` with ``decay_rank`` and ``tau``), ``norm`` (``all`` |
    ``head``), ``norm_eps``, ``gate_act`` (``sigmoid`` | ``silu``), ``buffers`` (a prefix for the workspace names)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["v_dim"])
        if self.dim > 512:
            raise ValueError("decay_linear_attention: the scan kernel holds heads of up to 512 key channels")
        self.activation = p.get("activation")
        if self.activation not in (None, "silu"):
            raise ValueError("decay_linear_attention: activation is None or 'silu'")
        self.q_scale = float(p.get("q_scale", 1.0))
        self.decay = p.get("decay", "head")
        if self.decay == "head":
            values = [float(v) for v in p["head_decay"]]
            if len(values) != self.nh:
                raise ValueError(f"decay_linear_attention: {len(values)} decays for {self.nh} heads")
            self.head_decay = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(device)
            self.rank, self.tau = 0, 1.0
        elif self.decay == "channel":
            self.head_decay = None
            self.rank = int(p["decay_rank"])
            self.tau = float(p["tau"])
            if self.tau <= 0 or self.rank <= 0:
                raise ValueError("decay_linear_attention: tau and decay_rank must be positive")
        else:
            raise ValueError("decay_linear_attention: decay is 'head' or 'channel'")
        self.norm = p.get("norm", "all")
        self.gate_act = p.get("gate_act", "sigmoid")
        if self.norm not in ("all", "head") or self.gate_act not in ("sigmoid", "silu"):
            raise ValueError("decay_linear_attention: norm is 'all' or 'head', gate_act 'sigmoid' or 'silu'")
        self.eps = float(p["norm_eps"])
        self.pre = str(p.get("buffers", ""))
        self.qk_size = self.nh * self.dim
        self.v_size = self.nh * self.vdim
        self.w_in = self.w_a1 = self.w_a2 = self.a2_bias = self.w_o = self.norm_w = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"q": TensorSpec((self.qk_size, self.hidden)), "k": TensorSpec((self.qk_size, self.hidden)),
             "v": TensorSpec((self.v_size, self.hidden)), "g": TensorSpec((self.v_size, self.hidden)),
             "o": TensorSpec((self.hidden, self.v_size)),
             "norm": TensorSpec((self.v_size if self.norm == "all" else self.vdim,), init="ones_jitter")}
        if self.decay == "channel":
            t["a1"] = TensorSpec((self.rank, self.hidden))
            t["a2"] = TensorSpec((self.qk_size, self.rank))
            t["a2.b"] = TensorSpec((self.qk_size,))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["q"], tensors["k"], tensors["v"], tensors["g"]]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()           # columns of the product: q | k | v | g
        self.w_o = tensors["o"].contiguous()
        w = tensors["norm"].to(torch.float32)
        self.norm_w = (w if self.norm == "all" else w.repeat(self.nh)).contiguous()
        if self.decay == "channel":
            self.w_a1 = tensors["a1"].contiguous()
            self.w_a2 = tensors["a2"].contiguous()
            self.a2_bias = tensors["a2.b"].to(torch.float32).contiguous()

    def input_rows(self) -> torch.Tensor:
        return self.w_in

    STATE_COLUMNS = 16          # the scan kernel keeps the state in blocks of that many contiguous columns (csrc/decay_scan.cu)

    def cache_need(self) -> StateNeed:
        blocks = -(-self.vdim // self.STATE_COLUMNS)
        return StateNeed((self.nh, blocks, self.STATE_COLUMNS, (self.dim + 3) // 4 * 4), torch.float32)

    def kernel_libraries(self):
        return ("decay_scan", "stream_ops", "gemm_simt")

    def forward(self, x, ctx, cache, writes_cache: bool, proj: Optional[torch.Tensor] = None):
        """``proj``: the columns ``q | k | v | g`` of a product someone else ran over ``input_rows()``."""
        if not writes_cache:
            raise ValueError("decay_linear_attention: a recurrent layer cannot read the state another call keeps")
        k = ops.kernels()
        n = x.shape[0]
        if proj is None:
            proj = ctx.buf(self.pre + "linear_in", (n, self.w_in.shape[0]), self.dtype)
            k.linear(x, self.w_in, proj)
        g0 = 2 * self.qk_size + self.v_size
        z = None
        if self.decay == "channel":
            low = ctx.buf(self.pre + "decay_low", (n, self.rank), self.dtype)
            k.linear(x, self.w_a1, low)
            z = ctx.buf(self.pre + "decay_z", (n, self.qk_size), torch.float32)
            k.linear(low, self.w_a2, z)
        heads = ctx.buf(self.pre + "scan_out", (n, self.v_size), torch.float32)
        k.decay_scan(proj, 0, self.qk_size, 2 * self.qk_size, cache.state, ctx.cu_q, ctx.state_slots, heads, num_heads=self.nh,
                     dim=self.dim, v_dim=self.vdim, activation=self.activation, q_scale=self.q_scale, head_decay=self.head_decay,
                     z=z, z_bias=self.a2_bias, tau=self.tau, max_q_len=ctx.max_q_len)
        normed = ctx.buf(self.pre + "scan_normed", (n, self.v_size), self.dtype)
        k.head_norm_gate_act(heads, self.norm_w, proj[:, g0: g0 + self.v_size], normed,
                             num_heads=1 if self.norm == "all" else self.nh, eps=self.eps, gate_act=self.gate_act)
        out = ctx.buf(self.pre + "mixer_out", (n, self.hidden), self.dtype)
        k.linear(normed, self.w_o, out)
        return out
