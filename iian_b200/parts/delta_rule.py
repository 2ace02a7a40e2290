"""The gated delta rule with a decay per key channel: a recurrent mixer whose state is a matrix per head.

``q = Wq h``, ``k = Wk h`` (kv_heads x dim), ``v = Wv h`` (heads x v_dim); head ``g`` uses the q / k head
``g // (heads / kv_heads)``.  Each of q, k, v passes a short causal convolution over time (one filter of ``conv`` taps per
channel, the last tap is the current token's, zeros before the start) and silu; q and k are then scaled to unit length per
head (``x / sqrt(sum x^2 + 1e-6)``), q also by ``dim^-1/2``.  Per head a write strength ``beta = sigmoid(Wb h)`` and per head
and key channel a decay ``g = exp(-exp(A_log) softplus(Wa2 (Wa1 h) + dt_bias))``.  With ``S`` [dim, v_dim] per head,

    S <- diag(g) S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q        (the read-out sees the token's own write)

Each head's ``o`` is divided by its root mean square, multiplied by a weight per column of the head (shared by the heads) and
by ``sigmoid(Wg2 (Wg1 h))``, and projected by ``Wo``.

The state (S in float32 and the convolution's last ``conv - 1`` inputs) lives in the request's state slot and is carried from
step to step; a step walks the tokens it brings in order.  ``Wq | Wk | Wv | Wb`` are one product; the decay's
pre-activation is a product with float32 output; unit lengths, sigmoid, softplus, exponentials and the recurrence are float32
in both dtypes (``csrc/delta_rule.cu``).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer

UNIT_LENGTH_FLOOR = 1e-6        # the design's constant under the root of a unit length (also fixed in the kernel)
MAX_TAPS = 8                    # what the kernels hold


def state_floats(num_heads: int, num_kv_heads: int, dim: int, v_dim: int, taps: int) -> int:
    """Floats of a request's state: S [heads, v_dim, dim], then the convolution's tail [taps - 1, channels]."""
    return num_heads * v_dim * dim + (taps - 1) * (2 * num_kv_heads * dim + num_heads * v_dim)


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim`` (query/key size per head), ``v_dim``, ``conv`` (taps
    of the short convolution), ``decay_rank`` and ``gate_rank`` (inner sizes of the two low-rank maps), ``norm_eps`` (of the
    heads' root mean square)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["v_dim"])
        self.taps = int(p["conv"])
        self.decay_rank = int(p["decay_rank"])
        self.gate_rank = int(p["gate_rank"])
        self.eps = float(p["norm_eps"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"gated_delta_rule: {self.nh} heads cannot share {self.nkv} query/key heads")
        if not 1 <= self.taps <= MAX_TAPS:
            raise ValueError(f"gated_delta_rule: the convolution has 1 to {MAX_TAPS} taps, got {self.taps}")
        if self.dim > 512:
            raise ValueError("gated_delta_rule: the scan kernel holds heads of up to 512 query/key entries")
        self.qk_size = self.nkv * self.dim
        self.v_size = self.nh * self.vdim
        self.channels = 2 * self.qk_size + self.v_size
        self.w_in = self.w_a1 = self.w_g1 = self.w_a2 = self.w_g2 = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"q": TensorSpec((self.qk_size, self.hidden)), "k": TensorSpec((self.qk_size, self.hidden)),
                "v": TensorSpec((self.v_size, self.hidden)),
                "q.conv": TensorSpec((self.qk_size, self.taps), init="ones_jitter"),
                "k.conv": TensorSpec((self.qk_size, self.taps), init="ones_jitter"),
                "v.conv": TensorSpec((self.v_size, self.taps), init="ones_jitter"),
                "b": TensorSpec((self.nh, self.hidden)), "A_log": TensorSpec((self.nh,), init="zeros_jitter"),
                "a1": TensorSpec((self.decay_rank, self.hidden)), "a2": TensorSpec((self.nh * self.dim, self.decay_rank)),
                "dt_bias": TensorSpec((self.nh * self.dim,), init="zeros_jitter"),
                "g1": TensorSpec((self.gate_rank, self.hidden)), "g2": TensorSpec((self.v_size, self.gate_rank)),
                "norm": TensorSpec((self.vdim,), init="ones_jitter"), "o": TensorSpec((self.hidden, self.v_size))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors[n] for n in ("q", "k", "v", "b")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.w_a1 = tensors["a1"].contiguous()
        self.w_g1 = tensors["g1"].contiguous()
        self.w_a2 = tensors["a2"].contiguous()
        self.w_g2 = tensors["g2"].contiguous()
        self.w_o = tensors["o"].contiguous()
        f32 = torch.float32
        self.conv_w = torch.cat([tensors["q.conv"].to(f32), tensors["k.conv"].to(f32), tensors["v.conv"].to(f32)], dim=0).contiguous()
        self.a_log = tensors["A_log"].to(f32).contiguous()
        self.dt_bias = tensors["dt_bias"].to(f32).contiguous()
        self.norm_w = tensors["norm"].to(f32).repeat(self.nh).contiguous()        # one weight per column of a head, every head alike

    def cache_need(self) -> StateNeed:
        return StateNeed((state_floats(self.nh, self.nkv, self.dim, self.vdim, self.taps),), torch.float32)

    def kernel_libraries(self):
        return ("delta_rule", "stream_ops", "gemm_simt")

    def forward(self, x, ctx, cache, writes_cache: bool):
        if not writes_cache:
            raise ValueError("gated_delta_rule: a recurrent layer cannot read the state another call keeps")
        k = ops.kernels()
        n = x.shape[0]
        proj = ctx.buf("delta_in", (n, self.w_in.shape[0]), self.dtype)
        k.linear(x, self.w_in, proj)
        b_off = self.channels
        a1 = ctx.buf("delta_a1", (n, self.decay_rank), self.dtype)
        k.linear(x, self.w_a1, a1)
        z = ctx.buf("delta_z", (n, self.nh * self.dim), torch.float32)       # the decay's pre-activation stays 32-bit
        k.linear(a1, self.w_a2, z)
        g1 = ctx.buf("delta_g1", (n, self.gate_rank), self.dtype)
        k.linear(x, self.w_g1, g1)
        gate = ctx.buf("delta_gate", (n, self.v_size), self.dtype)
        k.linear(g1, self.w_g2, gate)
        heads = ctx.buf("delta_heads", (n, self.v_size), torch.float32)
        k.delta_rule(proj, 0, b_off, z, self.conv_w, self.a_log, self.dt_bias, cache.state, ctx, heads, num_heads=self.nh,
                     num_kv_heads=self.nkv, dim=self.dim, v_dim=self.vdim)
        normed = ctx.buf("delta_normed", (n, self.v_size), self.dtype)
        k.head_norm_gate(heads, self.norm_w, gate, normed, num_heads=self.nh, eps=self.eps)
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.linear(normed, self.w_o, out)
        return out
