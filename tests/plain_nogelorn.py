"""A plain, slow implementation of the Nogelorn design: whole sequences, no cache, one function per mechanism.

It shares no code with ``iian_b200``: it takes a configuration (the ``config.json`` mapping) and the tensors by their
file names and computes with elementary torch operations on the CPU, in float64 by default, so that it can serve as the
oracle of the 32-bit and of the bfloat16 path.

Notation.  ``x`` [T, W] is the stream of one sequence, positions ``0 .. T-1``; ``e`` = table[token] * scale is what the
embedding leaves.  A layer has a norm before AND after each sub-layer:

    x' = x + n1b(mixer(n1(x)));    x'' = x' + n2b(ff(n2(x')))

with ``n(y) = y / sqrt(mean(y^2) + eps) * (1 + w)``.  A stretch of layers may run several times in a row with the same
weights; every run but the first starts with ``x <- x + e``.  The recurrent mixers are walked token by token and can be
given a state to start from and asked for the state they end with, so that a test can cut a sequence anywhere.
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


# ---- elementary pieces ------------------------------------------------------------------------------
product_rounding = None         # see plain_lekilix: a rounding applied around every matrix product, for sensitivity tests


def mm(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if product_rounding is None:
        return h @ w.T
    return product_rounding(product_rounding(h) @ w.T)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of this design: the stored weight sits around zero and one is added to it."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---- rotation ---------------------------------------------------------------------------------------
def base_frequencies(dims: int, base: float) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)


def banded_frequencies(dims: int, base: float, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies scaled by wavelength bands: short waves stay, long waves are divided by ``factor``, those between are
    blended linearly in ``original / wavelength``."""
    f = base_frequencies(dims, base)
    out = torch.empty_like(f)
    for i in range(f.numel()):
        fi = float(f[i])
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out[i] = fi
        elif wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def ramped_frequencies(dims: int, base: float, factor: float, original: float, fast: float, slow: float):
    """Frequencies blended by a ramp over the pair index, and the factor that multiplies cos and sin.  Returns ``(f, m)``."""
    f = base_frequencies(dims, base)

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(v: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """Rotate the first ``2 * len(freqs)`` entries of the last axis, entry i with entry i + len(freqs), by
    ``p * freqs[i]``; cos and sin are multiplied by ``magnitude``.  ``v`` is [T, heads, n]; the rest passes unchanged."""
    half = freqs.numel()
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    c = (torch.cos(ang) * magnitude).to(v.dtype)[:, None, :]
    s = (torch.sin(ang) * magnitude).to(v.dtype)[:, None, :]
    a, b = v[..., :half], v[..., half: 2 * half]
    out = v.clone()
    out[..., :half] = a * c - b * s
    out[..., half: 2 * half] = b * c + a * s
    return out


def rotation_of(rot: Optional[Mapping], kind: str):
    """``(freqs, magnitude)`` of a mixer's ``rot`` record; ``kind`` says how its ``scaling`` reads."""
    if rot is None:
        return None, 1.0
    dims, base = int(rot["dims"]), float(rot["base"])
    sc = rot.get("scaling")
    if sc is None:
        return base_frequencies(dims, base), 1.0
    if kind == "bands":
        return banded_frequencies(dims, base, float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])), 1.0
    return ramped_frequencies(dims, base, float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))


# ---- attention --------------------------------------------------------------------------------------
def visibility(q_pos: torch.Tensor, n_keys: int, size: Optional[int], keep_first: int = 0) -> torch.Tensor:
    """[Tq, n_keys] booleans: whether the query at position ``i`` sees key ``j``: never the future; inside the window, or
    one of the kept first keys."""
    i = q_pos.to(torch.long)[:, None]
    j = torch.arange(n_keys)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: Optional[int], keep_first: int = 0,
                     sink: Optional[torch.Tensor] = None, q_pos0: int = 0) -> torch.Tensor:
    """``q`` [Tq, H, d] at positions ``q_pos0 ..``, ``k`` [Tk, G, d], ``v`` [Tk, G, dv] at positions ``0 ..``.  Softmax over the
    visible keys; with ``sink`` [H] the denominator also holds ``exp(sink_h)`` (no key, no value, unscaled)."""
    tq, H, _ = q.shape
    G = k.shape[1]
    see = visibility(q_pos0 + torch.arange(tq), k.shape[0], size, keep_first)
    out = torch.zeros(tq, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~see, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h])
        p = torch.exp(s - m)
        den = p.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def window_attention_unit(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Softmax attention whose rotated q and k are divided by their root mean square per head (no weight)."""
    T = h.shape[0]
    H, G, d, dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = mm(h, w[pre + "q"]).view(T, H, d)
    k = mm(h, w[pre + "k"]).view(T, G, d)
    v = mm(h, w[pre + "v"]).view(T, G, dv)
    freqs, mag = rotation_of(cfg.get("rot"), "bands")
    pos = torch.arange(T)
    if freqs is not None:
        q, k = rotate_half(q, pos, freqs, mag), rotate_half(k, pos, freqs, mag)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    mask = cfg.get("mask") or {}
    o = masked_attention(q, k, v, float(cfg["scale"]), mask.get("size"))
    return mm(o.reshape(T, H * dv), w[pre + "o"])


def gated_sink_attention(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor) -> torch.Tensor:
    """Softmax attention with kept first keys, a sink in the denominator and one sigmoid gate per head."""
    T = h.shape[0]
    H, G, d, dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = mm(h, w[pre + "q"]).view(T, H, d)
    k = mm(h, w[pre + "k"]).view(T, G, d)
    v = mm(h, w[pre + "v"]).view(T, G, dv)
    freqs, mag = rotation_of(cfg.get("rot"), "ramp")
    pos = torch.arange(T)
    if freqs is not None:
        q, k = rotate_half(q, pos, freqs, mag), rotate_half(k, pos, freqs, mag)
    mask = cfg.get("mask") or {}
    o = masked_attention(q, k, v, float(cfg["scale"]), mask.get("size"), int(mask.get("keep_first", 0)), sink=w[pre + "sink"].to(h.dtype))
    gate = torch.sigmoid(mm(h, w[pre + "g"]))                      # [T, H]
    o = o * gate[:, :, None]
    return mm(o.reshape(T, H * dv), w[pre + "o"])


# ---- linear recurrences -----------------------------------------------------------------------------
def decayed_outer_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                       state: Optional[torch.Tensor] = None):
    """``S_t = diag(decay_t) S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` per head.  ``q``, ``k`` [T, H, d], ``v`` [T, H, dv],
    ``decay`` [T, H, d] (a decay per key channel; a decay per head is that number repeated).  Returns ``(o, S_T)``."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def lightning_mixer(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float, state=None, return_state=False):
    """Linear attention with one fixed decay per head; activations on q, k, v; one norm over all heads; sigmoid gate."""
    T = h.shape[0]
    H, d, dv = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = silu(mm(h, w[pre + "q"])).view(T, H, d)
    k = silu(mm(h, w[pre + "k"])).view(T, H, d)
    v = silu(mm(h, w[pre + "v"])).view(T, H, dv)
    decay = torch.tensor([float(x) for x in cfg["decay"]], dtype=h.dtype)[None, :, None].expand(T, H, d)
    o, S = decayed_outer_scan(q, k, v, decay, state)
    y = unit_rms(o.reshape(T, H * dv), eps) * w[pre + "norm"].to(h.dtype)
    y = y * torch.sigmoid(mm(h, w[pre + "g"]))
    out = mm(y, w[pre + "o"])
    return (out, S) if return_state else out


def channel_decay(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, tau: float) -> torch.Tensor:
    """``sigmoid(W2 (W1 h) + b)^(1/tau)``, one number per key channel."""
    z = mm(mm(h, w[pre + "a1"]), w[pre + "a2"]) + w[pre + "a2.b"].to(h.dtype)
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def gated_linear_attention(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float, state=None,
                           return_state=False):
    """Linear attention with a learned decay per key channel, a norm per head with a weight all heads share, a silu gate."""
    T = h.shape[0]
    H, d, dv = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = (mm(h, w[pre + "q"]) * d ** -0.5).view(T, H, d)
    k = mm(h, w[pre + "k"]).view(T, H, d)
    v = mm(h, w[pre + "v"]).view(T, H, dv)
    alpha = channel_decay(h, w, pre, float(cfg["tau"])).view(T, H, d)
    o, S = decayed_outer_scan(q, k, v, alpha, state)
    y = unit_rms(o, eps) * w[pre + "norm"].to(h.dtype)[None, None, :]
    y = y.reshape(T, H * dv) * silu(mm(h, w[pre + "g"]))
    out = mm(y, w[pre + "o"])
    return (out, S) if return_state else out


def side_by_side_mixer(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    left = window_attention_unit(cfg["left"], w, pre + "left.", h, eps)
    right = gated_linear_attention(cfg["right"], w, pre + "right.", h, eps)
    return float(cfg["left_scale"]) * left + float(cfg["right_scale"]) * right


# ---- feed-forward -----------------------------------------------------------------------------------
def gated_expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    return mm(silu(mm(h, w[pre + "gate"])) * mm(h, w[pre + "up"]), w[pre + "down"])


# A test that wants to know where a router's choice hangs on a hair sets this to a list; every call then appends, per token,
# the gap between the last chosen logit and the best one left out (infinity where every expert is chosen).
router_margins: Optional[list] = None


def router_choice(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, top: int):
    """``(ids [T, top], weights [T, top])``: the largest logits, softmax over the chosen ones only."""
    z = h @ w[pre + "router"].to(h.dtype).T + w[pre + "router.b"].to(h.dtype)
    vals, ids = torch.topk(z, top, dim=-1)
    if router_margins is not None:
        rest = torch.topk(z, top + 1, dim=-1).values[:, top] if top < z.shape[-1] else torch.full_like(vals[:, 0], -math.inf)
        router_margins.append(vals[:, top - 1] - rest)
    return ids, torch.softmax(vals, dim=-1)


def experts_feed_forward(cfg: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor) -> torch.Tensor:
    top = int(cfg["router"]["top"])
    ids, wts = router_choice(h, w, pre, top)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(top):
            out[t] += wts[t, c] * gated_expert(h[t: t + 1], w, f"{pre}e{int(ids[t, c])}.")[0]
    if cfg.get("shared") is not None:
        out = out + gated_expert(h, w, pre + "shared.")
    return out


# ---- the model --------------------------------------------------------------------------------------
def run_order(cfg: Mapping) -> List[tuple]:
    """(layer, whether a later run of the repeated stretch starts here)."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if lp is None:
        return [(i, False) for i in range(n)]
    start, stop, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    order = [(i, False) for i in range(start)]
    for r in range(times):
        order += [(i, r > 0 and i == start) for i in range(start, stop)]
    order += [(i, False) for i in range(stop, n)]
    return order


def mixer_of(layer: Mapping, w: Mapping[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    kind = layer["type"]
    if kind == "lightning":
        return lightning_mixer(layer["mixer"], w, pre, h, eps)
    if kind == "parallel":
        return side_by_side_mixer(layer["mixer"], w, pre, h, eps)
    if kind == "attention":
        return gated_sink_attention(layer["mixer"], w, pre, h)
    raise ValueError(kind)


def forward(cfg: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    e = w["embed"][tok] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = e.clone()
    streams = []
    for i, again in run_order(cfg):
        layer = cfg["layers"][i]
        if again:
            x = x + e
        h = offset_rms_norm(x, w[f"l{i}.norm1"], eps)
        x = x + offset_rms_norm(mixer_of(layer, w, f"l{i}.mix.", h, eps), w[f"l{i}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = offset_rms_norm(x, w[f"l{i}.norm2"], eps)
            x = x + offset_rms_norm(experts_feed_forward(layer["mlp"], w, f"l{i}.mlp.", h), w[f"l{i}.norm2b"], eps)
        streams.append(x.clone())
    logits = offset_rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits
