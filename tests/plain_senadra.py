"""A plain, slow implementation of the Senadra design: whole sequences, no cache, one function per mechanism.

It shares no code with ``iian_b200``: it takes a configuration (the ``config.json`` mapping) and the tensors by their
file names and computes with elementary torch operations on the CPU, in float64 by default, so that it can serve as the
oracle of the 32-bit and of the bfloat16 path.

Notation.  ``x`` [T, W] is the stream of one sequence, positions ``0 .. T-1``, ``m`` the model's residual factor.  A layer
is ``x += m mixer(norm1 x)``; ``x += m ff(norm2 x)``; ``x += m unit_rms(P (gelu(G x) * e_i)) * w`` with ``e_i`` the layer's
slice of a second embedding row of the token.  Mixers: attention inside chunks of positions with a logarithmic distance
penalty and normalised values; attention over a low-rank latent with a shared rotated key part and a latent for the
queries; a delta-rule recurrence with a decay per key channel.  The logits pass a tanh cap.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional

import torch

from plain_qwen3 import read_safetensors


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# What a matrix product's input and result pass through: nothing.  A test that wants to know how far 16-bit products alone
# move the logits sets this to a rounding function for the time of a call.
product_rounding = None


def mm(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``h W^T`` (weights are stored [out, in])."""
    if product_rounding is None:
        return h @ w.T
    return product_rounding(product_rounding(h) @ w.T)


# ---- elementary pieces ------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def unit_length(x: torch.Tensor, floor: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + floor)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """Positive side ``softplus(p) z^2 + z / 2``; the other ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``."""
    ap = softplus(p)
    an = 0.5 + softplus(q)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(neg) - neg) + 0.5 * z)


def tanh_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotate the first ``dims`` entries of the last axis, entry 2i with entry 2i+1, by ``p * base^(-2i/dims)``.
    ``v`` is [T, heads, n]; entries from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]        # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_mask(t: int) -> torch.Tensor:
    i = torch.arange(t)
    return i[None, :] <= i[:, None]


def chunk_mask(t: int, size: Optional[int]) -> torch.Tensor:
    """[i, j] true iff j <= i and both lie in the same chunk of ``size`` positions counted from 0."""
    i = torch.arange(t)
    vis = i[None, :] <= i[:, None]
    if size:
        vis = vis & ((i[None, :] // size) == (i[:, None] // size))
    return vis


def masked_softmax(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j taps[c, j] x[t - (n - 1) + j, c]`` with zeros before the start (the last tap is the current token's)."""
    n = taps.shape[1]
    pad = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + pad[j: j + x.shape[0]] * taps[:, j][None, :]
    return y


# ---- mixers ------------------------------------------------------------------------------------------
def keys_values(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float):
    """What a chunked-attention layer puts into its cache: keys as projected, values divided by their root mean square."""
    T = h.shape[0]
    k = mm(h, t[pre + "k"]).view(T, mc["kv_heads"], mc["dim"])
    v = unit_rms(mm(h, t[pre + "v"]).view(T, mc["kv_heads"], mc["vdim"]), eps)
    return k, v


def distance_penalty(t: int, r1: torch.Tensor, r2: torch.Tensor) -> torch.Tensor:
    """[heads, i, j]: ``r1_h ln(1 + r2_h (i - j))`` (zero where j > i)."""
    i = torch.arange(t, dtype=r1.dtype)
    d = torch.clamp(i[:, None] - i[None, :], min=0)
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * d[None])


def chunked_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float, kv) -> torch.Tensor:
    """``kv``: the (keys, values) this layer reads: its own or those of the layer named by ``kv_from``."""
    T = h.shape[0]
    H, G, D, V = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = mm(h, t[pre + "q"]).view(T, H, D)
    k, v = kv
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)            # head g reads KV head g // rep
    vh = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kh) * mc["scale"]
    scores = scores - distance_penalty(T, t[pre + "r1"].to(h.dtype), t[pre + "r2"].to(h.dtype))
    size = (mc.get("mask") or {}).get("size")
    p = masked_softmax(scores, chunk_mask(T, size)[None])
    o = torch.einsum("hij,jhd->ihd", p, vh).reshape(T, H * V)
    o = o * torch.sigmoid(mm(h, t[pre + "g"]))
    return mm(o, t[pre + "o"])


def latent_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float) -> torch.Tensor:
    """Keys and values in their EXPANDED form: per head ``[Wuk c ; kr]`` and ``Wuv c``."""
    T = h.shape[0]
    H, D, R, V, rank = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(mm(h, t[pre + "dq"]), t[pre + "dq.norm"], eps)
    q = mm(cq, t[pre + "uq"]).view(T, H, D + R)
    dkv = mm(h, t[pre + "dkv"])
    c = rms_norm(dkv[:, :rank], t[pre + "dkv.norm"], eps)
    kr = dkv[:, rank:].view(T, 1, R)
    rot = mc["rot"]
    qr = rotate_pairs(q[..., D:], pos, rot["dims"], rot["base"])
    kr = rotate_pairs(kr, pos, rot["dims"], rot["base"])
    kn = mm(c, t[pre + "uk"]).view(T, H, D)
    v = mm(c, t[pre + "uv"]).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :D], kn) + torch.einsum("ihd,jd->hij", qr, kr[:, 0])) * mc["scale"]
    p = masked_softmax(scores, causal_mask(T)[None])
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * V)
    o = o * torch.sigmoid(mm(h, t[pre + "g"]))
    return mm(o, t[pre + "o"])


def channel_delta(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float, state=None,
                  return_state: bool = False):
    """The delta rule with a decay per key channel, token by token.  ``state``: (S [heads, dim, vdim], tail of the
    convolution's inputs [taps - 1, channels]) of the tokens before, or None at the start of a sequence."""
    T = h.shape[0]
    H, G, D, V = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    raw = torch.cat([mm(h, t[pre + "q"]), mm(h, t[pre + "k"]), mm(h, t[pre + "v"])], dim=1)
    taps = torch.cat([t[pre + "q.conv"], t[pre + "k.conv"], t[pre + "v.conv"]], dim=0).to(h.dtype)
    n = taps.shape[1]
    if state is None:
        S = torch.zeros(H, D, V, dtype=h.dtype)
        tail = torch.zeros(n - 1, raw.shape[1], dtype=h.dtype)
    else:
        S, tail = state[0].clone(), state[1]
    ext = torch.cat([tail, raw], dim=0)
    conv = causal_conv(ext, taps)[n - 1:]
    if product_rounding is not None:
        conv = product_rounding(conv)
    act = silu(conv)
    q = unit_length(act[:, : G * D].view(T, G, D)) * D ** -0.5
    k = unit_length(act[:, G * D: 2 * G * D].view(T, G, D))
    v = act[:, 2 * G * D:].view(T, H, V)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(mm(h, t[pre + "b"]))                                     # [T, H]
    step = softplus(mm(mm(h, t[pre + "a1"]), t[pre + "a2"]) + t[pre + "dt_bias"].to(h.dtype)).view(T, H, D)
    decay = torch.exp(-torch.exp(t[pre + "A_log"].to(h.dtype))[None, :, None] * step)      # [T, H, D]
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        S = decay[i][:, :, None] * S
        u = beta[i][:, None] * (v[i] - torch.einsum("hdv,hd->hv", S, k[i]))
        S = S + k[i][:, :, None] * u[:, None, :]
        o[i] = torch.einsum("hdv,hd->hv", S, q[i])
    o = unit_rms(o, eps) * t[pre + "norm"].to(h.dtype)[None, None, :]
    gate = torch.sigmoid(mm(mm(h, t[pre + "g1"]), t[pre + "g2"])).view(T, H, V)
    y = mm((o * gate).reshape(T, H * V), t[pre + "o"])
    if return_state:
        return y, (S, ext[ext.shape[0] - (n - 1):])
    return y


# ---- the rest of a layer ----------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    a = t[pre + "act"].to(h.dtype)
    return mm(xielu(mm(h, t[pre + "up"]), a[0], a[1]), t[pre + "down"])


def token_side(x: torch.Tensor, e: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    """What the per-layer token input adds (before the residual factor): ``unit_rms(P (gelu(G x) * e)) * w``."""
    g = gelu_tanh(mm(x, t[pre + "gate"])) * e
    return rms_norm(mm(g, t[pre + "proj"]), t[pre + "norm"].to(x.dtype), eps)


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the stream after every layer [L, T, W])."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    tok = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    m = cfg.get("residual_mult", 1.0)
    x = t["embed"][tok]
    side = cfg.get("token_side")
    kept: Dict[int, tuple] = {}
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}."
        mc = lc["mixer"]
        h = rms_norm(x, t[pre + "norm1"], eps)
        if lc["type"] == "attention":
            src = mc.get("kv_from")
            if src is None:
                kept[i] = keys_values(h, t, pre + "mix.", mc, eps)
                kv = kept[i]
            else:
                kv = kept[src]
            y = chunked_attention(h, t, pre + "mix.", mc, eps, kv)
        elif lc["type"] == "latent_attention":
            y = latent_attention(h, t, pre + "mix.", mc, eps)
        elif lc["type"] == "channel_delta":
            y = channel_delta(h, t, pre + "mix.", mc, eps)
        else:
            raise ValueError(lc["type"])
        x = x + m * y
        if lc.get("mlp") is not None:
            x = x + m * dense_ff(rms_norm(x, t[pre + "norm2"], eps), t, pre + "mlp.")
        if side is not None:
            d = side["dim"]
            e = t["side.embed"][tok][:, i * d: (i + 1) * d]
            x = x + m * token_side(x, e, t, pre + "side.", eps)
        layers.append(x)
    logits = mm(rms_norm(x, t["final.norm"], eps), t["head"])
    if cfg.get("logit_softcap") is not None:
        logits = tanh_cap(logits, cfg["logit_softcap"])
    if return_layers:
        return logits, torch.stack(layers)
    return logits
