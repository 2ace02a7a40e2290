"""A rotated attention mixer whose sliding window may keep the first keys of the sequence.

``q = Wq h`` (heads x dim), ``k = Wk h`` (kv_heads x dim), ``v = Wv h`` (kv_heads x v_dim), no biases.  The first ``rot``
entries of every head of q and k are rotated by the position (entry i with entry i + rot / 2; the part in ``position`` gives
the frequencies, possibly rescaled for long contexts, and a magnitude on cos and sin).  With ``unit_norm`` every head of q and
k is THEN divided by its root mean square (no weight).  Head ``g`` reads KV head ``g // (heads / kv_heads)``;

    s_ij = (q_i . k_j) * scale,      key j visible to position i  iff  j <= i and (i - j < window or j < keep_first)

(kept keys keep their true positions: they are rotated and cached like all others).  Softmax over the visible keys; with
``sink`` the denominator also holds ``exp(sink_g)``, a learned number per head without key or value.  With ``head_gate`` head
g's output is multiplied by ``sigmoid(Wg h)_g``, one number per head read from the same input as the projections.  ``Wo`` on
the concatenated heads.

``Wq | Wk | Wv | Wg`` are one product (``input_rows``); a mixer that holds this one beside another may run that product
itself, together with the other's, and hand over the columns (``forward(..., proj=...)``).  The cache is a K/V page cache whose
value cells have ``v_dim`` entries.  A layer with kept keys gives no pages back (its first pages stay needed for ever and
the page groups free from the front); a plain window does.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, POSITIONS, register_mixer


@register_mixer("window_attention")
class WindowAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_dim``, ``scale``, ``window`` (None or keys
    visible, the query's own included), ``keep_first`` (0 or how many first keys stay visible), ``sink`` (bool),
    ``head_gate`` (bool), ``unit_norm`` (bool) with ``unit_norm_eps``, ``position`` (a PartSpec: ``rotary``,
    ``scaled_rotary`` or ``none``; pairs (i, i + rot / 2)), ``buffers`` (a prefix for the workspace names, for two of these in
    one layer)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_dim", self.hd))
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"window_attention: {self.nh} heads cannot share {self.nkv} KV heads")
        if max(self.hd, self.vd) > 512:
            raise ValueError("window_attention: heads of up to 512 entries")
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window_attention: window must be positive or None")
        self.keep_first = int(p.get("keep_first", 0) or 0)
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ValueError("window_attention: keep_first needs a window and cannot be negative")
        self.has_sink = bool(p.get("sink", False))
        self.has_gate = bool(p.get("head_gate", False))
        self.unit_norm = bool(p.get("unit_norm", False))
        self.eps = float(p.get("unit_norm_eps", 0.0))
        self.position = POSITIONS.build(p.get("position") or _NONE, dtype, device)
        self.rot = int(getattr(self.position, "dim", 0) or 0)
        if self.rot > self.hd:
            raise ValueError(f"window_attention: the position encoding rotates {self.rot} entries of a head of {self.hd}")
        if self.rot and getattr(self.position, "style", 0) != 0:
            raise ValueError("window_attention: pairs are (i, i + rot / 2)")
        self.pre = str(p.get("buffers", ""))
        self.q_size = self.nh * self.hd
        self.k_size = self.nkv * self.hd
        self.v_size = self.nkv * self.vd
        self.o_size = self.nh * self.vd
        self.w_in = self.w_o = self.sink = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"q": TensorSpec((self.q_size, self.hidden)), "k": TensorSpec((self.k_size, self.hidden)),
             "v": TensorSpec((self.v_size, self.hidden)), "o": TensorSpec((self.hidden, self.o_size))}
        if self.has_sink:
            t["sink"] = TensorSpec((self.nh,), init="zeros_jitter")
        if self.has_gate:
            t["g"] = TensorSpec((self.nh, self.hidden))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.has_gate else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()           # columns of the product: q | k | v | g
        self.w_o = tensors["o"].contiguous()
        if self.has_sink:
            self.sink = tensors["sink"].to(torch.float32).contiguous()

    def input_rows(self) -> torch.Tensor:
        """The stacked matrix of everything this mixer multiplies with its input."""
        return self.w_in

    def cache_need(self) -> KVNeed:
        keep = int(self.window) if self.window is not None and not self.keep_first else None
        return KVNeed(self.nkv, self.hd, keep, self.vd if self.vd != self.hd else None)

    def _fast(self) -> bool:
        return self.dtype == torch.bfloat16 and self.hd == self.vd and self.hd in (64, 128) and self.scale > 0

    def kernel_libraries(self):
        return ("window_attention", "gemm_simt") + (("attention_mma",) if self._fast() else ()) \
            + (("attention_tc",) if self._fast() and self.hd == 128 else ())

    def graph_plan(self, num_seqs: int, max_ctx: int):
        k = ops.kernels()
        if not hasattr(k, "window_attention_plan"):
            return None
        return k.window_attention_plan(num_seqs, self.nh, self.nkv, self.hd, self.vd, self.scale, max_ctx, self.window,
                                       self.keep_first, self.dtype)

    def forward(self, x, ctx, cache, writes_cache: bool, proj: Optional[torch.Tensor] = None, plan=None):
        """``proj``: the columns ``q | k | v | g`` of a product someone else ran over ``input_rows()`` (a column slice)."""
        if not writes_cache:
            raise ValueError("window_attention: a layer of this kind fills its own cache")
        k = ops.kernels()
        n = x.shape[0]
        if proj is None:
            proj = ctx.buf(self.pre + "window_in", (n, self.w_in.shape[0]), self.dtype)
            k.linear(x, self.w_in, proj)
        meta = ctx.page_meta(cache.group)
        table = self.position.table64(ctx) if self.rot else None
        q = ctx.buf(self.pre + "q", (n, self.nh, self.hd), self.dtype)
        k.rotate_unit_store(proj, 0, self.q_size, self.q_size + self.k_size, q, cache.k, cache.v, table, meta.slots,
                            num_heads=self.nh, num_kv_heads=self.nkv, k_dim=self.hd, v_dim=self.vd, rot_dim=self.rot, eps=self.eps,
                            unit_norm=self.unit_norm)
        g0 = self.q_size + self.k_size + self.v_size
        gate = proj[:, g0: g0 + self.nh] if self.has_gate else None
        attn = ctx.buf(self.pre + "attn", (n, self.o_size), self.dtype)
        if plan is None:
            plan = ctx.graph_plan(self)
        k.window_attention(q.view(n, self.q_size), cache.k, cache.v, attn, meta, num_heads=self.nh, num_kv_heads=self.nkv,
                           k_dim=self.hd, v_dim=self.vd, scale=self.scale, window=self.window, keep_first=self.keep_first,
                           sink=self.sink, gate=gate, gate_per_head=True, **({"n_split": plan["n_split"]} if plan else {}))
        out = ctx.buf(self.pre + "mixer_out", (n, self.hidden), self.dtype)
        k.linear(attn, self.w_o, out)
        return out


from ..config.spec import PartSpec  # noqa: E402

_NONE = PartSpec("none")
