"""Attention whose keys and values are read out of one cached low-rank latent per token.

Per token: ``q = Wq h`` (per head ``dim`` plain and ``rot`` rotated entries); ``Wdkv h`` gives ``rank + rot`` numbers, the
first ``rank`` RMS-normalised into the latent ``c``, the last ``rot`` one rotated key part ``kr`` that every head shares.
Head ``g`` has keys ``(Wuk_g c_j, kr_j)`` and values ``Wuv_g c_j``.  Neither is ever formed here.  Since
``q_g . (Wuk_g c_j) = (Wuk_g^T q_g) . c_j``, the query moves into latent space (``qa_g = Wuk_g^T q_g``), every head
scores the SAME cached row ``(c_j, kr_j)``: ``s_j = (qa_g . c_j + qr_g . kr_j) * scale``, and the weighted sum of the
latents is lifted once per query: ``o_g = Wuv_g (sum_j p_j c_j)``.  The cache holds ``rank + rot`` numbers per token and
a step reads each cached row once for all heads.

The softmax may carry a sink per head (a logit with no key and no value that joins the denominator), keys may be
limited to a window, and the rotation (either pairing, over the first ``rot.dim`` of the ``rot`` entries) is a
``rotary`` position part.  The queries may come through a latent of their own (``q_rank``): ``cq = RMSnorm(Wdq h)``,
``q = Wuq cq``; the concatenated heads may be multiplied by ``sigmoid(Wg h)`` before ``Wo`` (``output_gate``).

A mixer may also be asked for further rows of the same input (``extra_rows``): whatever else reads the mixer's input
through a matrix (a gate of the residual) is stacked under ``Wq | Wdkv`` so that one product serves all; the extra
columns come back beside the mixer's output.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Mixer, POSITIONS, RowNeed, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``dim`` (plain query/key entries per head), ``rot_dim`` (rotated ones),
    ``v_dim``, ``kv_rank``, ``scale``, ``norm_eps`` (of the latent's RMS norm), ``window`` (None or keys visible),
    ``sink`` (bool), ``position`` (a PartSpec: ``rotary`` over the first ``dim`` of the rotated entries, or ``none``);
    optional ``q_rank`` (None or the size of the queries' latent; tensors ``dq``, ``dq.norm``, ``uq`` instead of ``q``) and
    ``output_gate`` (bool; tensor ``g``)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p["v_dim"])
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["norm_eps"])
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("latent_attention: window must be positive or None")
        self.has_sink = bool(p.get("sink", False))
        self.position = POSITIONS.build(p["position"], dtype, device)
        if not getattr(self.position, "fused", False):
            raise ValueError("latent_attention: the position encoding must be a rotation (or none)")
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else None
        self.has_gate = bool(p.get("output_gate", False))
        if getattr(self.position, "dim", 0) > self.rot:
            raise ValueError(f"latent_attention: position encoding rotates {self.position.dim} of {self.rot} rotated entries")
        self.q_size = self.nh * (self.dim + self.rot)
        self.dkv_size = self.rank + self.rot
        self.width = self.rank + self.rot
        self.extra_rows: Optional[torch.Tensor] = None
        self.w_uq = self.q_norm_w = None
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.norm_w = self.sink = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {
            "dkv": TensorSpec((self.dkv_size, self.hidden)),
            "dkv.norm": TensorSpec((self.rank,), init="ones_jitter"),
            "uk": TensorSpec((self.nh * self.dim, self.rank)),
            "uv": TensorSpec((self.nh * self.vdim, self.rank)),
            "o": TensorSpec((self.hidden, self.nh * self.vdim)),
        }
        if self.q_rank is None:
            t["q"] = TensorSpec((self.q_size, self.hidden))
        else:
            t["dq"] = TensorSpec((self.q_rank, self.hidden))
            t["dq.norm"] = TensorSpec((self.q_rank,), init="ones_jitter")
            t["uq"] = TensorSpec((self.q_size, self.q_rank))
        if self.has_sink:
            t["sink"] = TensorSpec((self.nh,))
        if self.has_gate:
            t["g"] = TensorSpec((self.nh * self.vdim, self.hidden))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        # the first product's rows: the queries (or their latent) | the down-projected latent and key part | the gate | extras
        self._w_q, self._w_dkv = tensors["q" if self.q_rank is None else "dq"], tensors["dkv"]
        self._w_gate = tensors["g"] if self.has_gate else None
        if self.q_rank is not None:
            self.w_uq = tensors["uq"].contiguous()
            self.q_norm_w = tensors["dq.norm"].to(torch.float32).contiguous()
        self._stack()
        self.w_uk = tensors["uk"].contiguous()
        self.w_uv = tensors["uv"].contiguous()
        self.w_o = tensors["o"].contiguous()
        self.norm_w = tensors["dkv.norm"].to(torch.float32).contiguous()
        self.sink = tensors["sink"].to(torch.float32).contiguous() if self.has_sink else None

    def _stack(self) -> None:
        ws = [self._w_q, self._w_dkv] + ([self._w_gate] if self._w_gate is not None else []) \
            + ([self.extra_rows] if self.extra_rows is not None else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()

    def stack_rows(self, rows: torch.Tensor) -> None:
        """Further rows [m, hidden] to be multiplied with the mixer's input in the same product (call after ``bind``)."""
        self.extra_rows = rows
        self._stack()

    def cache_need(self) -> RowNeed:
        return RowNeed(self.width, int(self.window) if self.window is not None else None)

    def kernel_libraries(self):
        return ("latent_attention", "gemm_simt") + (("latent_attention_mma",) if self.dtype == torch.bfloat16 else ()) \
            + (("residual_ops",) if self.q_rank is not None else ()) + (("stream_ops",) if self.has_gate else ())

    def graph_plan(self, num_seqs: int, max_ctx: int):
        """The number of key parts of the tensor-core kernel is part of a captured graph (its grid)."""
        k = ops.kernels()
        if not hasattr(k, "latent_attention_parts"):
            return None
        return {"parts": k.latent_attention_parts(num_seqs, 1, self.nh, max_ctx, self.window)}

    def forward(self, x, ctx, cache, writes_cache: bool, with_extra: bool = False):
        """``x`` [N, hidden] in the activation dtype.  Returns the mixer's output [N, hidden], or with ``with_extra`` the
        pair (output, the extra columns [N, m] of the stacked product, a column slice)."""
        k = ops.kernels()
        n = x.shape[0]
        pos = self.position
        n_extra = self.extra_rows.shape[0] if self.extra_rows is not None else 0
        q_cols = self.q_size if self.q_rank is None else self.q_rank
        n_gate = self.nh * self.vdim if self.has_gate else 0
        total = q_cols + self.dkv_size + n_gate + n_extra
        qd = ctx.buf("latent_in", (n, total), self.dtype)
        k.linear(x, self.w_in, qd)
        meta = ctx.page_meta(cache.group)
        q_cat = ctx.buf("latent_q", (n, self.nh, self.width), self.dtype)
        queries = None
        if self.q_rank is not None:        # the queries through their latent: norm, then the up-projection
            cq = ctx.buf("latent_cq", (n, self.q_rank), self.dtype)
            k.rms_norm_rows(qd[:, : self.q_rank], self.q_norm_w, self.eps, cq)
            queries = ctx.buf("latent_queries", (n, self.q_size), self.dtype)
            k.linear(cq, self.w_uq, queries)
        # the latent's norm, the rotations, the cache write; rotated query parts go to the back of q_cat's rows
        k.latent_prep(qd, 0, q_cols, cache.rows if writes_cache else None, q_cat, self.norm_w,
                      pos.inv_freq64, ctx.positions, meta.slots if writes_cache else None,
                      num_heads=self.nh, dim=self.dim, rot=self.rot, rank=self.rank, rot_dims=pos.dim, eps=self.eps,
                      queries=queries, style=getattr(pos, "style", 0))
        # qa_g = Wuk_g^T q_g into the front of q_cat's rows
        k.head_linear(qd if queries is None else queries, 0, self.dim + self.rot, self.w_uk, self.dim * self.rank, self.rank, 1,
                      q_cat.view(n, self.nh * self.width), 0, self.width, num_heads=self.nh, n_in=self.dim, n_out=self.rank)
        lat = ctx.buf("latent_ctx", (n, self.nh, self.rank), self.dtype)
        if hasattr(k, "latent_attention_mma_ok") and k.latent_attention_mma_ok(q_cat, cache.rows, self.rank):
            plan = ctx.graph_plan(self)
            k.latent_attention_mma(q_cat, cache.rows, lat, self.sink, meta, num_heads=self.nh, rank=self.rank, scale=self.scale,
                                   window=self.window, parts=plan["parts"] if plan else None)
        else:
            k.latent_attention(q_cat, cache.rows, lat, self.sink, meta, num_heads=self.nh, rank=self.rank, scale=self.scale,
                               window=self.window)
        # o_g = Wuv_g (sum_j p_j c_j)
        heads = ctx.buf("latent_heads", (n, self.nh * self.vdim), self.dtype)
        k.head_linear(lat.view(n, self.nh * self.rank), 0, self.rank, self.w_uv, self.vdim * self.rank, 1, self.rank,
                      heads, 0, self.vdim, num_heads=self.nh, n_in=self.rank, n_out=self.vdim)
        if self.has_gate:
            gated = ctx.buf("latent_gated", (n, self.nh * self.vdim), self.dtype)
            k.sigmoid_mul(heads, qd[:, q_cols + self.dkv_size: q_cols + self.dkv_size + n_gate], gated)
            heads = gated
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.linear(heads, self.w_o, out)
        if with_extra:
            return out, (qd[:, q_cols + self.dkv_size + n_gate:] if n_extra else None)
        return out
