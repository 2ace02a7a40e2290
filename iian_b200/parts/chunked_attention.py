"""An attention mixer without rotation: positions enter through the mask and through a penalty on distance.

``q = Wq h`` (heads x dim), ``k = Wk h`` (kv_heads x dim), ``v = Wv h`` (kv_heads x v_dim; a value may have another size
than a key).  Each head's value is divided by its root mean square (``value_norm``; it is cached so).  Head ``g`` reads KV
head ``g // (heads / kv_heads)``; the score of key ``j`` for position ``i`` is

    s_ij = (q_i . k_j) * scale - r1_g ln(1 + r2_g (i - j))            (``distance_penalty``: two numbers per head)

and key ``j`` is visible iff ``j <= i`` and, with ``chunk`` = c, ``i // c == j // c`` (chunks are counted from position 0 of
the sequence, wherever a prompt was cut); with ``window`` = w instead, iff ``i - j < w``.  Softmax over the visible keys; the
concatenated heads are multiplied by ``sigmoid(Wg h)`` (``output_gate``) and projected by ``Wo``.

``Wq | Wk | Wv | Wg`` are one product.  A call that reads the cache another call filled (``writes_cache=False``) has no key
and value projections of its own: its product is ``Wq | Wg``.  The cache is a K/V page cache whose value cells have
``v_dim`` entries (``KVNeed.v_dim``).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, register_mixer


@register_mixer("chunked_attention")
class ChunkedAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_dim``, ``scale``, ``chunk`` (None or the
    chunk's size), ``window`` (None or keys visible; not together with ``chunk``), ``value_norm`` (bool) with
    ``value_norm_eps``, ``distance_penalty`` (bool), ``output_gate`` (bool), ``owns_kv`` (bool, default True: False for a
    layer that only ever reads another layer's cache and has no key / value projections)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_dim", self.hd))
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"chunked_attention: {self.nh} heads cannot share {self.nkv} KV heads")
        self.scale = float(p["scale"])
        self.chunk = p.get("chunk")
        self.window = p.get("window")
        if self.chunk is not None and self.window is not None:
            raise ValueError("chunked_attention: either a chunk or a window")
        for name, v in (("chunk", self.chunk), ("window", self.window)):
            if v is not None and int(v) <= 0:
                raise ValueError(f"chunked_attention: {name} must be positive or None")
        self.value_norm = bool(p.get("value_norm", False))
        self.eps = float(p.get("value_norm_eps", 0.0))
        self.penalty = bool(p.get("distance_penalty", False))
        self.has_gate = bool(p.get("output_gate", False))
        self.owns_kv = bool(p.get("owns_kv", True))
        self.q_size = self.nh * self.hd
        self.k_size = self.nkv * self.hd
        self.v_size = self.nkv * self.vd
        self.o_size = self.nh * self.vd
        self.w_in = self.w_o = self.r1 = self.r2 = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"q": TensorSpec((self.q_size, self.hidden)), "o": TensorSpec((self.hidden, self.o_size))}
        if self.owns_kv:
            t["k"] = TensorSpec((self.k_size, self.hidden))
            t["v"] = TensorSpec((self.v_size, self.hidden))
        if self.penalty:
            t["r1"] = TensorSpec((self.nh,), init="ones_jitter")
            t["r2"] = TensorSpec((self.nh,), init="ones_jitter")
        if self.has_gate:
            t["g"] = TensorSpec((self.o_size, self.hidden))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        # column layout of the stacked product: q | g | k | v, so that a reader of another layer's cache uses the front
        ws = [tensors["q"]] + ([tensors["g"]] if self.has_gate else []) + ([tensors["k"], tensors["v"]] if self.owns_kv else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        if self.penalty:
            self.r1 = tensors["r1"].to(torch.float32).contiguous()
            self.r2 = tensors["r2"].to(torch.float32).contiguous()

    def cache_need(self) -> KVNeed:
        keep = int(self.window) if self.window is not None else None
        return KVNeed(self.nkv, self.hd, keep, self.vd if self.vd != self.hd else None)

    def kernel_libraries(self):
        fast = self.dtype == torch.bfloat16 and self.hd == self.vd and self.hd in (64, 128) and self.scale > 0
        return ("chunked_attention", "gemm_simt") + (("attention_mma",) if fast else ()) + (("attention_tc",) if fast and self.hd == 128 else ())

    def graph_plan(self, num_seqs: int, max_ctx: int):
        k = ops.kernels()
        if not hasattr(k, "chunked_attention_plan"):
            return None
        return k.chunked_attention_plan(num_seqs, self.nh, self.nkv, self.hd, self.vd, self.scale, max_ctx, self.chunk, self.window,
                                        self.dtype)

    def forward(self, x, ctx, cache, writes_cache: bool):
        if writes_cache and not self.owns_kv:
            raise ValueError("chunked_attention: a layer without key / value projections cannot fill a cache")
        k = ops.kernels()
        n = x.shape[0]
        front = self.q_size + (self.o_size if self.has_gate else 0)
        w = self.w_in if writes_cache else self.w_in[:front]
        proj = ctx.buf("chunked_in", (n, w.shape[0]), self.dtype)
        k.linear(x, w, proj)
        meta = ctx.page_meta(cache.group)
        if writes_cache:
            k.kv_store_normed(proj, front, front + self.k_size, cache.k, cache.v, meta.slots, num_kv_heads=self.nkv, k_dim=self.hd,
                              v_dim=self.vd, eps=self.eps, norm_values=self.value_norm)
        gate = proj[:, self.q_size: front] if self.has_gate else None
        attn = ctx.buf("attn", (n, self.o_size), self.dtype)
        plan = ctx.graph_plan(self)
        k.chunked_attention(proj[:, : self.q_size], cache.k, cache.v, attn, meta, num_heads=self.nh, num_kv_heads=self.nkv,
                            k_dim=self.hd, v_dim=self.vd, scale=self.scale, chunk=self.chunk, window=self.window, r1=self.r1,
                            r2=self.r2, gate=gate, **({"n_split": plan["n_split"]} if plan else {}))
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.linear(attn, self.w_o, out)
        return out
