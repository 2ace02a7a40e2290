"""The benchmark workloads: model shapes by name, device-timed decode and prefill with their rooflines, and
continuous batching of many requests through the scheduler.

``iian bench --shape ...`` and the repository's ``bench.py`` both call this module.  The method is the
reference's (tests/e2e/bench-batch.cpp:45-84, src/iian/cli/cmd_bench.cpp:18-96): random weights, seeded uniform
random token ids, greedy, ``ignore_eos``; wall clock for the scheduler-driven runs (TTFT = time to a request's
first token, TPOT = mean time between its tokens), CUDA events around the step function for the device-timed
figures.  Rooflines: a decode step has to read every weight it uses once and the cache of its live requests
(HBM bytes / time against the measured copy bandwidth); a prefill step's flops / time against the measured
bfloat16 matrix-product peak.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
import statistics
import time
from typing import Dict, List, Optional, Sequence

# name -> config.json keys of the shape (random weights; no checkpoint is read)
SHAPES: Dict[str, dict] = {
    "tinyA": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
                  max_position_embeddings=128, tie_word_embeddings=True),
    "tinyB": dict(vocab_size=503, hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=8,
                  num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
                  max_position_embeddings=256, tie_word_embeddings=False),
    "0.6b": dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                 max_position_embeddings=40960, tie_word_embeddings=True),
    "8b": dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
               max_position_embeddings=40960, tie_word_embeddings=False),
    "32b": dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                max_position_embeddings=40960, tie_word_embeddings=False),
}


def _galodra_shape(width, heads, layers, ff=0, experts=0, top=0, expert_ff=0, vocab=32768, window=4096):
    mixer = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
             "rot": {"dims": 64, "base": 10000.0}, "mask": {"size": window}}
    mlp = ({"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}} if experts
           else {"kind": "dense", "ff": ff})
    return {"architecture": "Galodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": dict(mlp)} for _ in range(layers)]}


def _qwen3_shape(hidden, heads, layers, inter, vocab=32768):
    return dict(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                tie_word_embeddings=True)


# Galodra shapes with layer sizes of real models (latent rank 512 + 64 rotated, heads of 128 + 64, window 4096), eight
# layers each, and beside each the Qwen3 dense shape of equal width, heads, layers and (active) feed-forward size.
GALODRA_SHAPES: Dict[str, dict] = {
    "g2k-dense": _galodra_shape(2048, 16, 8, ff=8192),
    "g2k-moe": _galodra_shape(2048, 16, 8, experts=64, top=6, expert_ff=1408),
    "g4k-dense": _galodra_shape(4096, 32, 8, ff=12288),
}
EQUAL_QWEN3: Dict[str, dict] = {
    "g2k-dense": _qwen3_shape(2048, 16, 8, 8192),
    "g2k-moe": _qwen3_shape(2048, 16, 8, 6 * 1408),
    "g4k-dense": _qwen3_shape(4096, 32, 8, 12288),
}


def _lekilix_shape(width, heads, ff=0, experts=0, top=0, expert_ff=0, vocab=32768, window=4096):
    """Six layers, memory and attention in turn, of which the first two run twice (eight layer runs, as the Qwen3 shape beside
    it has eight layers): attention heads of 128 on 8 key/value heads, memories of half as many heads, 128 deep and 256 wide."""
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                          "rot": {"dims": 64, "base": 500000.0}, "mask": {"size": window}}}
    mem = {"type": "mlstm", "mixer": {"heads": heads // 2, "dim": 128, "vdim": 256, "gate_cap": 15.0}}
    mlp = ({"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0}, "router": {"experts": experts, "top": top}} if experts
           else {"kind": "dense", "ff": ff})
    return {"architecture": "Lekilix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [dict(mem if i % 2 == 0 else att, mlp=dict(mlp)) for i in range(6)]}


# Lekilix shapes with layer sizes of real models, and beside each the Qwen3 dense shape of equal width, heads, layer runs and
# (active) feed-forward size.
LEKILIX_SHAPES: Dict[str, dict] = {
    "l2k-dense": _lekilix_shape(2048, 16, ff=8192),
    "l2k-moe": _lekilix_shape(2048, 16, experts=64, top=6, expert_ff=1408),
    "l4k-dense": _lekilix_shape(4096, 32, ff=12288),
}
EQUAL_QWEN3.update({"l2k-dense": _qwen3_shape(2048, 16, 8, 8192), "l2k-moe": _qwen3_shape(2048, 16, 8, 6 * 1408),
                    "l4k-dense": _qwen3_shape(4096, 32, 8, 12288)})


def _senadra_shape(width, heads, ff, vocab=32768, chunk=2048):
    """Eight layers -- chunked attention, delta rule, latent attention, a reader of the first layer's keys and values, delta
    rule, latent attention, chunked attention, delta rule: attention heads of 128 on 8 key/value heads; recurrences of as many
    value heads 128 wide on half as many query/key heads 128 deep, four taps; latents of 512 + 64 rotated behind a query
    latent of 1,536; a second per-token input of 256 per layer; an ungated feed-forward 1.5 times as wide as the gated one
    of the Qwen3 shape beside it (equal weights)."""
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                          "mask": {"size": chunk}}}
    reader = {"type": "attention", "mixer": dict(att["mixer"], kv_from=0)}
    rec = {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4,
                                              "decay_rank": 64, "gate_rank": 64}}
    lat = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512,
                                                 "q_rank": 1536, "scale": 192 ** -0.5, "rot": {"dims": 64, "base": 10000.0}}}
    order = [att, rec, lat, reader, rec, lat, att, rec]
    return {"architecture": "Senadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "token_side": {"dim": 256}, "logit_softcap": 30.0,
            "layers": [dict(type=l["type"], mixer=dict(l["mixer"]), mlp={"kind": "dense", "ff": ff}) for l in order]}


# Senadra shapes with layer sizes of real models, and beside each the Qwen3 dense shape of equal width, heads, layers and
# feed-forward weights.
SENADRA_SHAPES: Dict[str, dict] = {
    "s2k": _senadra_shape(2048, 16, 12288),
    "s4k": _senadra_shape(4096, 32, 18432),
}
EQUAL_QWEN3.update({"s2k": _qwen3_shape(2048, 16, 8, 8192), "s4k": _qwen3_shape(4096, 32, 8, 12288)})
def _nogelorn_shape(width, heads, experts, top, expert_ff, vocab=32768, window=4096, keep=128):
    """Six layers of which the first two run twice (eight layer runs, as the shapes beside it): a side-by-side layer (sliding-
    window attention of 128-wide heads on 8 key/value heads beside linear attention with a decay per key channel, half as
    many heads, 128 deep and 128 wide), attention with kept first keys, a sink and a gate per head, and linear attention with
    a constant decay per head (half as many heads, 128 deep and 256 wide: the state of the Lekilix memory beside it);
    experts with one more that every token uses (so ``top`` + 1 are active)."""
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                          "rot": {"dims": 64, "base": 1000000.0,
                                                  "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                                          "mask": {"size": window, "keep_first": keep}}}
    left = {"heads": heads, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": window},
            "rot": {"dims": 128, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    par = {"type": "parallel", "mixer": {"left": left, "left_scale": 0.6, "right_scale": 0.9,
                                         "right": {"heads": heads // 2, "dim": 128, "vdim": 128, "tau": 16.0, "decay_rank": 16}}}
    nh = heads // 2
    lin = {"type": "lightning", "mixer": {"heads": nh, "dim": 128, "vdim": 256,
                                          "decay": [math.exp(-0.5 * (i + 1) / nh) for i in range(nh)]}}
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": expert_ff}}
    order = [par, att, lin, att, lin, att]
    return {"architecture": "Nogelorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [dict(type=l["type"], mixer=copy.deepcopy(l["mixer"]), mlp=copy.deepcopy(mlp)) for l in order]}


# Nogelorn shapes with layer sizes of real models; beside each the Lekilix shape of equal width, heads, layer runs and active
# experts (its closest relative in the framework: a looped stretch, experts, recurrences beside windowed attention with a sink)
# and the Qwen3 dense shape of equal active size.
NOGELORN_SHAPES: Dict[str, dict] = {
    "n2k-moe": _nogelorn_shape(2048, 16, 64, 5, 1408),
    "n4k-moe": _nogelorn_shape(4096, 32, 64, 5, 2048),
}
EQUAL_QWEN3.update({"n2k-moe": _qwen3_shape(2048, 16, 8, 6 * 1408), "n4k-moe": _qwen3_shape(4096, 32, 8, 6 * 2048)})
EQUAL_LEKILIX: Dict[str, dict] = {
    "n2k-moe": _lekilix_shape(2048, 16, experts=64, top=6, expert_ff=1408),
    "n4k-moe": _lekilix_shape(4096, 32, experts=64, top=6, expert_ff=2048),
}
DESIGN_SHAPES = {"galodra": GALODRA_SHAPES, "lekilix": LEKILIX_SHAPES, "senadra": SENADRA_SHAPES, "nogelorn": NOGELORN_SHAPES}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks(root: Optional[str] = None):
    """Measured copy bandwidth and bfloat16 product peak of this pool's GPUs if ``MEASURED_PEAKS.json`` lies in
    ``root`` (the repository), else the stated fallback: ``(peaks, "measured" | "fallback")``."""
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def shape_config(name: str, layers: Optional[int] = None):
    from ..models.qwen3 import qwen3_config_from_dict
    if name in GALODRA_SHAPES:
        from ..models.galodra import galodra_config_from_dict
        raw = dict(GALODRA_SHAPES[name])
        if layers:
            raw["layers"] = raw["layers"][:layers]
        return galodra_config_from_dict(raw)
    if name in LEKILIX_SHAPES:
        from ..models.lekilix import lekilix_config_from_dict
        raw = dict(LEKILIX_SHAPES[name])
        if layers:
            raw["layers"] = raw["layers"][:layers]
            raw["loop"] = None if layers < raw["loop"]["stop"] else raw["loop"]
        return lekilix_config_from_dict(raw)
    if name in SENADRA_SHAPES:
        from ..models.senadra import senadra_config_from_dict
        raw = dict(SENADRA_SHAPES[name])
        if layers:
            raw["layers"] = raw["layers"][:layers]
        return senadra_config_from_dict(raw)
    if name in NOGELORN_SHAPES:
        from ..models.nogelorn import nogelorn_config_from_dict
        raw = dict(NOGELORN_SHAPES[name])
        if layers:
            raw["layers"] = raw["layers"][:layers]
            raw["loop"] = None if layers < raw["loop"]["stop"] else raw["loop"]
        return nogelorn_config_from_dict(raw)
    try:
        raw = dict(SHAPES[name])
    except KeyError:
        known = list(SHAPES) + list(GALODRA_SHAPES) + list(LEKILIX_SHAPES) + list(SENADRA_SHAPES) + list(NOGELORN_SHAPES)
        raise ValueError(f"unknown shape '{name}' ({' | '.join(known)})") from None
    if layers:
        raw["num_hidden_layers"] = layers
    return qwen3_config_from_dict(raw)


def random_model(name: str, dtype: str = "bfloat16", device="cuda:0", seed: int = 0, layers: Optional[int] = None):
    """The shape ``name`` with random weights N(0, 0.02) and norm weights 1, drawn on the device."""
    from ..config.registry import get_architecture
    from ..engine.model import Model
    cfg = shape_config(name, layers)
    arch = ("Galodra" if name in GALODRA_SHAPES else "Lekilix" if name in LEKILIX_SHAPES else "Senadra" if name in SENADRA_SHAPES
            else "Nogelorn" if name in NOGELORN_SHAPES else "Qwen3ForCausalLM")
    return Model.from_random(get_architecture(arch), cfg, seed=seed, dtype=dtype, device=device, norm_jitter=0.0)


def accounting_for(cfg, dtype_bytes: int = 2):
    """Bytes and flops of a step for a configuration of any built-in architecture."""
    if type(cfg).__name__ == "NogelornConfig":
        return NogelornAccounting(cfg, dtype_bytes)
    if hasattr(cfg, "embedding_scale"):
        return LekilixAccounting(cfg, dtype_bytes)
    if hasattr(cfg, "residual_mult"):
        return SenadraAccounting(cfg, dtype_bytes)
    return GalodraAccounting(cfg, dtype_bytes) if hasattr(cfg, "postln_alpha") else Accounting(cfg, dtype_bytes)


class Accounting:
    """Bytes and flops of a dense Qwen3 step, from the configuration."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg = cfg
        self.layer_w = cfg.hidden_size * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * cfg.hidden_size \
            + 3 * cfg.hidden_size * cfg.intermediate_size
        self.head_w = cfg.vocab_size * cfg.hidden_size
        self.weight_bytes_step = dtype_bytes * (cfg.num_hidden_layers * self.layer_w + self.head_w)
        self.kv_bytes_token = cfg.num_hidden_layers * 2 * cfg.kv_size * dtype_bytes

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        return self.weight_bytes_step + batch * ctx_avg * self.kv_bytes_token

    def prefill_flops(self, tokens: int) -> float:
        c = self.cfg
        return 2.0 * tokens * c.num_hidden_layers * self.layer_w + 2.0 * self.head_w \
            + c.num_hidden_layers * 4.0 * c.q_size * tokens * (tokens + 1) / 2


class GalodraAccounting:
    """Bytes and flops of a Galodra step.  A decode step reads every dense weight once, of routed experts those that the
    batch is expected to reach (``E (1 - (1 - top / E)^batch)`` of E), and of the latent cache the rows inside each
    layer's window."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg, self.b = cfg, dtype_bytes
        self.head_w = cfg.vocab * cfg.width

    def _layer(self, lc, batch: int):
        """(weights read by a step of ``batch`` tokens, weights a token multiplies with) of one layer."""
        w, m = self.cfg.width, lc.mixer
        mix = w * (m.heads * (m.dim + m.rot_dim) + m.kv_rank + m.rot_dim + w) + m.heads * (m.dim + m.vdim) * m.kv_rank \
            + w * m.heads * m.vdim
        if lc.mlp is None:
            return mix, mix
        if lc.mlp.kind == "dense":
            ff = 3 * w * lc.mlp.ff + w * w
            return mix + ff, mix + ff
        e, top = lc.mlp.experts, lc.mlp.top
        reached = e * (1.0 - (1.0 - top / e) ** batch)
        shared = (e + w) * w
        return mix + shared + reached * 3 * w * lc.mlp.ff, mix + shared + top * 3 * w * lc.mlp.ff

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        total = self.head_w * self.b
        for lc in self.cfg.layers:
            total += self._layer(lc, batch)[0] * self.b
            keys = min(ctx_avg, lc.mixer.window) if lc.mixer.window else ctx_avg
            total += batch * keys * (lc.mixer.kv_rank + lc.mixer.rot_dim) * self.b
        return total

    def prefill_flops(self, tokens: int) -> float:
        total = 2.0 * self.head_w
        for lc in self.cfg.layers:
            m = lc.mixer
            total += 2.0 * tokens * self._layer(lc, 1)[1]
            w = m.window or tokens
            pairs = tokens * (tokens + 1) / 2 if tokens <= w else w * (w + 1) / 2 + (tokens - w) * w
            total += 2.0 * m.heads * (2 * m.kv_rank + m.rot_dim) * pairs
        return total


class LekilixAccounting:
    """Bytes and flops of a Lekilix step, layer run by layer run (a layer of the looped stretch counts every time it runs: its
    weights do not stay in the L2 between two runs at these sizes).  A decode step reads every dense weight once per run, of
    the experts those that the batch is expected to reach, of the K/V cache the cells inside the window, and reads and
    writes every memory's float32 state."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg, self.b = cfg, dtype_bytes
        self.head_w = cfg.vocab * cfg.width

    def _layer(self, lc, batch: int):
        """(weights read by a step of ``batch`` tokens, weights a token multiplies with) of one layer run."""
        w, m = self.cfg.width, lc.mixer
        if lc.type == "attention":
            mix = w * (2 * m.heads + m.kv_heads) * m.dim + m.heads * m.dim * w
        else:
            mix = w * (2 * m.heads * m.dim + 2 * m.heads * m.vdim + 2 * m.heads) + m.heads * m.vdim * w
        if lc.mlp is None:
            return mix, mix
        if lc.mlp.kind == "dense":
            return mix + 3 * w * lc.mlp.ff, mix + 3 * w * lc.mlp.ff
        e, top = lc.mlp.experts, lc.mlp.top
        reached = e * (1.0 - (1.0 - top / e) ** batch)
        return mix + reached * 3 * w * lc.mlp.ff, mix + top * 3 * w * lc.mlp.ff

    def _runs(self):
        return [(self.cfg.layers[i], starts) for i, starts in self.cfg.run_order()]

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        total = self.head_w * self.b
        for lc, starts in self._runs():
            total += (self._layer(lc, batch)[0] + (2 * self.cfg.width ** 2 if starts else 0)) * self.b
            m = lc.mixer
            if lc.type == "attention":
                keys = min(ctx_avg, m.window) if m.window else ctx_avg
                total += batch * keys * 2 * m.kv_heads * m.dim * self.b
            else:
                total += batch * 2 * m.heads * (m.dim * m.vdim + m.dim) * 4
        return total

    def prefill_flops(self, tokens: int) -> float:
        total = 2.0 * self.head_w
        for lc, starts in self._runs():
            m = lc.mixer
            total += 2.0 * tokens * (self._layer(lc, 1)[1] + (2 * self.cfg.width ** 2 if starts else 0))
            if lc.type == "attention":
                w = m.window or tokens
                pairs = tokens * (tokens + 1) / 2 if tokens <= w else w * (w + 1) / 2 + (tokens - w) * w
                total += 4.0 * m.heads * m.dim * pairs
            else:
                total += 4.0 * tokens * m.heads * m.dim * (m.vdim + 1)         # the update and the read-out of every token
        return total


class NogelornAccounting:
    """Bytes and flops of a Nogelorn step, layer run by layer run (a layer of the looped stretch counts every time it runs).  A
    decode step reads every dense weight once per run, of the experts those that the batch is expected to reach plus the
    shared one, of a K/V cache the cells inside the window and the kept first ones, and reads and writes every recurrence's
    float32 state."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg, self.b = cfg, dtype_bytes
        self.head_w = cfg.vocab * cfg.width

    @staticmethod
    def _attention_w(w, m, gate: bool):
        return w * (m.heads + m.kv_heads) * m.dim + w * m.kv_heads * m.vdim + m.heads * m.vdim * w + (w * m.heads if gate else 0)

    @staticmethod
    def _linear_w(w, m, rank: int = 0):
        return w * (2 * m.heads * m.dim + 2 * m.heads * m.vdim) + m.heads * m.vdim * w + rank * (w + m.heads * m.dim)

    def _layer(self, lc, batch: int):
        """(weights read by a step of ``batch`` tokens, weights a token multiplies with) of one layer run."""
        w, m = self.cfg.width, lc.mixer
        if lc.type == "attention":
            mix = self._attention_w(w, m, True)
        elif lc.type == "lightning":
            mix = self._linear_w(w, m)
        else:
            mix = self._attention_w(w, m.left, False) + self._linear_w(w, m.right, m.right.rank)
        if lc.mlp is None:
            return mix, mix
        if lc.mlp.kind == "dense":
            return mix + 3 * w * lc.mlp.ff, mix + 3 * w * lc.mlp.ff
        e, top = lc.mlp.experts, lc.mlp.top
        reached = e * (1.0 - (1.0 - top / e) ** batch)
        fixed = w * e + 3 * w * lc.mlp.shared_ff
        return mix + fixed + reached * 3 * w * lc.mlp.ff, mix + fixed + top * 3 * w * lc.mlp.ff

    def _runs(self):
        return [self.cfg.layers[i] for i, _ in self.cfg.run_order()]

    @staticmethod
    def _members(lc):
        """(attention members, recurrent members) of a layer."""
        if lc.type == "attention":
            return [lc.mixer], []
        if lc.type == "lightning":
            return [], [lc.mixer]
        return [lc.mixer.left], [lc.mixer.right]

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        total = self.head_w * self.b
        for lc in self._runs():
            total += self._layer(lc, batch)[0] * self.b
            att, rec = self._members(lc)
            for m in att:
                keys = min(ctx_avg, m.window + m.keep_first) if m.window else ctx_avg
                total += batch * keys * m.kv_heads * (m.dim + m.vdim) * self.b
            for m in rec:
                total += batch * 2 * m.heads * m.dim * m.vdim * 4
        return total

    def prefill_flops(self, tokens: int) -> float:
        total = 2.0 * self.head_w
        for lc in self._runs():
            total += 2.0 * tokens * self._layer(lc, 1)[1]
            att, rec = self._members(lc)
            for m in att:
                w = m.window or tokens
                pairs = tokens * (tokens + 1) / 2 if tokens <= w else w * (w + 1) / 2 + (tokens - w) * (w + m.keep_first)
                total += 2.0 * m.heads * (m.dim + m.vdim) * pairs
            for m in rec:
                total += 4.0 * tokens * m.heads * m.dim * m.vdim               # the update and the read-out of every token
        return total


class SenadraAccounting:
    """Bytes and flops of a Senadra step.  A decode step reads every weight once, of a chunked layer's K/V cache the cells of
    the query's chunk, of a latent cache every row, and reads and writes every recurrence's float32 state; of the second
    embedding table a token reads one row."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg, self.b = cfg, dtype_bytes
        self.head_w = cfg.vocab * cfg.width

    def _layer(self, lc) -> float:
        """Weights of one layer."""
        w, m = self.cfg.width, lc.mixer
        if lc.type == "attention":
            mix = w * (m.heads * m.dim + m.heads * m.vdim) + m.heads * m.vdim * w
            if m.kv_from is None:
                mix += w * m.kv_heads * (m.dim + m.vdim)
        elif lc.type == "latent_attention":
            q = w * m.q_rank + m.q_rank * m.heads * (m.dim + m.rot_dim) if m.q_rank else w * m.heads * (m.dim + m.rot_dim)
            mix = q + w * (m.kv_rank + m.rot_dim) + m.heads * (m.dim + m.vdim) * m.kv_rank + 2 * w * m.heads * m.vdim
        else:
            mix = w * (2 * m.kv_heads * m.dim + m.heads * m.vdim + m.heads) + w * (m.decay_rank + m.gate_rank) \
                + m.decay_rank * m.heads * m.dim + m.gate_rank * m.heads * m.vdim + m.heads * m.vdim * w
        if lc.mlp is not None:
            mix += 2 * w * lc.mlp.ff
        return mix + 2 * w * self.cfg.side_dim

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        total = self.head_w * self.b
        for lc in self.cfg.layers:
            total += self._layer(lc) * self.b
            m = lc.mixer
            if lc.type == "attention":
                keys = min(ctx_avg, (m.chunk + 1) / 2) if m.chunk else ctx_avg
                total += batch * keys * m.kv_heads * (m.dim + m.vdim) * self.b
            elif lc.type == "latent_attention":
                total += batch * ctx_avg * (m.kv_rank + m.rot_dim) * self.b
            else:
                total += batch * 2 * m.heads * m.dim * m.vdim * 4
        return total

    def prefill_flops(self, tokens: int) -> float:
        total = 2.0 * self.head_w
        for lc in self.cfg.layers:
            m = lc.mixer
            total += 2.0 * tokens * self._layer(lc)
            if lc.type == "attention":
                c = m.chunk or tokens
                full, rest = divmod(tokens, c)
                pairs = full * c * (c + 1) / 2 + rest * (rest + 1) / 2
                total += 2.0 * m.heads * (m.dim + m.vdim) * pairs
            elif lc.type == "latent_attention":
                total += 2.0 * m.heads * (2 * m.kv_rank + m.rot_dim) * tokens * (tokens + 1) / 2
            else:
                total += 6.0 * tokens * m.heads * m.dim * m.vdim          # S^T k, the update and the read-out of every token
        return total


class TokenSource:
    def __init__(self, vocab: int, seed: int = 1234):
        import torch
        self.vocab = vocab
        self.gen = torch.Generator().manual_seed(seed)

    def take(self, n: int) -> List[int]:
        import torch
        return torch.randint(5, max(6, self.vocab - 5), (n,), generator=self.gen).tolist()


def prefill_requests(runner, source: TokenSource, batch: int, prompt_len: int, budget: int = 2048):
    """``batch`` requests with ``prompt_len`` random tokens each in the cache (several prompts to a step)."""
    from ..engine.runner import StepEntry
    mgr = runner.manager
    caches = []
    for _ in range(batch):
        rc = mgr.new_request()
        mgr.allot_state(rc)
        caches.append(rc)
    per_step = max(1, budget // prompt_len)
    for i in range(0, batch, per_step):
        ents = []
        for rc in caches[i:i + per_step]:
            if not mgr.allocate(rc, 0, prompt_len):
                raise RuntimeError("the cache is too small for this batch of prompts")
            ents.append(StepEntry(rc, source.take(prompt_len), 0, []))
        runner.step(ents)
    return caches


def measure_decode(runner, source: TokenSource, batch: int, prompt_len: int, warmup: int, steps: int) -> dict:
    """Decode ``batch`` requests from prompts of ``prompt_len`` tokens: ``warmup`` untimed steps, then ``steps`` steps of
    the step function plus the on-device argmax between two CUDA events.  Each step streams every weight from HBM
    (they exceed the L2 many times), so nothing survives in the L2 between timed iterations."""
    import torch
    from .. import ops
    from ..engine.runner import StepEntry
    kern, mgr, dev = ops.kernels(), runner.manager, runner.device
    caches = prefill_requests(runner, source, batch, prompt_len)
    out = torch.empty(batch, dtype=torch.int32, device=dev)
    toks = source.take(batch)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pos, launches0 = prompt_len, 0
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = runner.launches
            start.record()
        ents = []
        for rc, t in zip(caches, toks):
            if not mgr.allocate(rc, pos, 1):
                raise RuntimeError("out of cache pages while decoding")
            ents.append(StepEntry(rc, [t], pos, [0]))
        logits = runner.step(ents)
        kern.argmax(logits, out)
        pos += 1
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = runner.launches - launches0 + steps
    for rc in caches:
        mgr.free(rc)
    return {"batch": batch, "ms_per_step": ms, "tokens_per_s": batch / (ms * 1e-3), "launches": int(launches),
            "ctx_avg": prompt_len + warmup + (steps + 1) / 2}


def measure_prefill(runner, source: TokenSource, tokens: int, warmup: int = 3, repeats: int = 5) -> dict:
    """One prompt of ``tokens`` tokens as one step; the median of ``repeats`` runs after ``warmup`` runs."""
    import torch
    from ..engine.runner import StepEntry
    mgr = runner.manager
    toks = source.take(tokens)
    times = []
    for i in range(warmup + repeats):
        rc = mgr.new_request()
        mgr.allot_state(rc)
        if not mgr.allocate(rc, 0, tokens):
            raise RuntimeError("the cache is too small for this prompt")
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s_ev.record()
        runner.step([StepEntry(rc, toks, 0, [tokens - 1])])
        e_ev.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s_ev.elapsed_time(e_ev))
        mgr.free(rc)
    ms = statistics.median(times)
    return {"tokens": tokens, "ms": ms, "tokens_per_s": tokens / (ms * 1e-3)}


def decode_and_prefill_points(model, batches: Sequence[int], prompt_len: int, steps: int, warmup: int,
                              prefill_tokens: Sequence[int], context_len: int, peaks: dict, cuda_graphs: bool = True) -> dict:
    """Decode at every batch of ``batches`` and prefill at every length of ``prefill_tokens`` for one model, with the
    roofline fractions: ``{"decode": {B: {...}}, "prefill": {T: {...}}}``."""
    from ..config.engine import EngineConfig, SchedulerConfig
    from ..engine.engine import Engine
    acc = accounting_for(model.config)
    max_b = max(batches) if batches else 1
    per_req = prompt_len + warmup + steps + 48
    longest = max([per_req] + list(prefill_tokens))
    max_len = -(-max(context_len, longest + 16) // 16) * 16       # whole pages
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=max_len, kv_cache_tokens=max(max_len, max_b * per_req),
                        block_size=16, enable_prefix_caching=False, warmup=True, cuda_graphs=cuda_graphs,
                        sched=SchedulerConfig(max_num_seqs=max(1, max_b), max_num_batched_tokens=max(2048, longest)))
    engine = Engine(model, ecfg)
    src = TokenSource(model.vocab_size)
    out = {"decode": {}, "prefill": {}, "engine": engine}
    for b in batches:
        r = measure_decode(engine.runner, src, b, prompt_len, warmup, steps)
        nbytes = acc.decode_bytes(b, r["ctx_avg"])
        r["hbm_gbs"] = nbytes / (r["ms_per_step"] * 1e-3) / 1e9
        r["roofline_frac"] = r["hbm_gbs"] / peaks["hbm_gbs"]
        r["bytes_per_step"] = nbytes
        out["decode"][b] = r
    for t in prefill_tokens:
        r = measure_prefill(engine.runner, src, t, warmup=max(2, min(warmup, 3)))
        flops = acc.prefill_flops(t)
        r["tflops"] = flops / (r["ms"] * 1e-3) / 1e12
        r["frac"] = r["tflops"] / peaks["bf16_tflops"]
        out["prefill"][t] = r
    return out


# ---- continuous batching of many requests (BASELINE's Qwen3-0.6B workload) -----------------------------------
def serving_requests(vocab: int, n_requests: int, prompt_range=(16, 4096), output_range=(16, 512), shared_prefix: int = 512,
                     shared_fraction: float = 0.5, seed: int = 7):
    """``n_requests`` (prompt, output length) pairs: prompt lengths uniform in ``prompt_range``, output lengths
    uniform in ``output_range``, uniform random token ids; ``shared_fraction`` of the requests begin with the same
    ``shared_prefix`` tokens (their length is then at least that prefix plus one token)."""
    rng = random.Random(seed)
    prefix = [rng.randrange(5, max(6, vocab - 5)) for _ in range(shared_prefix)]
    out = []
    for i in range(n_requests):
        n = rng.randint(*prompt_range)
        n_out = rng.randint(*output_range)
        shares = rng.random() < shared_fraction
        if shares:
            n = max(n, shared_prefix + 1)
            toks = prefix + [rng.randrange(5, max(6, vocab - 5)) for _ in range(n - shared_prefix)]
        else:
            toks = [rng.randrange(5, max(6, vocab - 5)) for _ in range(n)]
        out.append((toks, n_out, shares))
    return out


def run_serving(engine, requests, check_alone: int = 0) -> dict:
    """Submit every request at once, step until all are finished (wall clock), and report throughput, latencies,
    prefix-cache hit rate, preemptions and the peak cache usage.  ``check_alone``: afterwards (untimed) that many of
    the requests are run again one at a time and their greedy tokens compared with what they produced in the crowd
    (``alone_mismatches`` counts requests whose tokens differ before their first near-tie cannot be told: in
    bfloat16 a different batch changes the rounding, so only the agreeing prefix length is reported)."""
    import torch
    from ..sampling.params import SamplingParams
    reqs = []
    for toks, n_out, _ in requests:
        reqs.append(engine.submit(toks, SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True)))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    peak_usage, steps = 0.0, 0
    while engine.step():               # False once no request is left to run
        steps += 1
        if steps % 8 == 0:
            peak_usage = max(peak_usage, engine.cache.usage)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    st = engine.stats()
    n_prompt = sum(len(t) for t, _, _ in requests)
    n_gen = sum(r.n_output for r in reqs)
    errors = sum(1 for r in reqs if not r.is_finished or r.finish_reason.value == "error")
    out = {"requests": len(reqs), "wall_s": secs, "steps": steps, "prompt_tokens": n_prompt, "generated_tokens": n_gen,
           "total_tok_s": (n_prompt + n_gen) / secs, "gen_tok_s": n_gen / secs, "prompt_tok_s": n_prompt / secs,
           "ttft_ms": st.ttft_ms_avg, "tpot_ms": st.tpot_ms_avg,
           "prefix_queries": st.prefix_cache_queries, "prefix_hits": st.prefix_cache_hits,
           "prefix_hit_rate": st.prefix_cache_hits / st.prefix_cache_queries if st.prefix_cache_queries else 0.0,
           "cached_prompt_tokens": st.cached_prompt_tokens, "preemptions": st.preemptions, "kv_usage_peak": peak_usage,
           "errors": errors}
    if check_alone:
        step = max(1, len(reqs) // check_alone)
        agree, total, full = 0, 0, 0
        for i in list(range(0, len(reqs), step))[:check_alone]:
            toks, n_out, _ = requests[i]
            n_cmp = min(n_out, 32)
            r = engine.submit(toks, SamplingParams(temperature=0.0, max_tokens=n_cmp, ignore_eos=True))
            while not r.is_finished:
                engine.step()
            a, b = r.output_tokens, reqs[i].output_tokens[:n_cmp]
            k = 0
            while k < len(a) and k < len(b) and a[k] == b[k]:
                k += 1
            agree += k
            total += n_cmp
            full += int(k == n_cmp)
        out["alone_checked"] = check_alone
        out["alone_identical"] = full
        out["alone_agreeing_token_share"] = agree / total if total else 1.0
    return out


def serving_workload(shape: str = "0.6b", n_requests: int = 256, kv_cache_tokens: int = 0, max_num_seqs: int = 64,
                     max_num_batched_tokens: int = 2048, seed: int = 7, check_alone: int = 8, device="cuda:0",
                     prompt_range=(16, 4096), output_range=(16, 512), shared_prefix: int = 512, model=None) -> dict:
    """BASELINE's continuous-batching workload: ``n_requests`` requests, prompts U[16, 4096], outputs U[16, 512],
    half sharing a 512-token prefix, through the scheduler with prefix reuse on and a cache small enough that
    requests are preempted (by default a third of what the running requests could hold at their longest)."""
    from ..config.engine import EngineConfig, SchedulerConfig
    from ..engine.engine import Engine
    model = model or random_model(shape, "bfloat16", device)
    max_len = prompt_range[1] + output_range[1] + 16
    if not kv_cache_tokens:
        kv_cache_tokens = max(max_len, max_num_seqs * max_len // 3)
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=max_len, kv_cache_tokens=kv_cache_tokens, block_size=16,
                        enable_prefix_caching=True, warmup=True, cuda_graphs=True,
                        sched=SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens))
    engine = Engine(model, ecfg)
    reqs = serving_requests(model.vocab_size, n_requests, prompt_range, output_range, shared_prefix, 0.5, seed)
    out = run_serving(engine, reqs, check_alone)
    out.update({"shape": shape, "kv_cache_tokens": kv_cache_tokens, "max_num_seqs": max_num_seqs,
                "max_num_batched_tokens": max_num_batched_tokens})
    return out


# ---- one design beside another of equal size ------------------------------------------------------------------------
def design_comparison(names: Sequence[str], batches: Sequence[int], prefill_tokens: Sequence[int], prompt_len: int, steps: int,
                      warmup: int, peaks: dict, device="cuda:0", cuda_graphs: bool = True, design: str = "galodra") -> dict:
    """Decode and prefill throughput of each named shape of ``design`` and of the Qwen3 shape of equal size, random weights:
    ``{name: {design: {...}, "qwen3": {...}}}`` with tokens/s and roofline fractions per point."""
    import gc
    import torch
    from ..config.registry import get_architecture
    from ..engine.model import Model
    from ..models.qwen3 import qwen3_config_from_dict
    out = {}
    for name in names:
        row = {}
        for side in (design, "lekilix", "qwen3") if design == "nogelorn" else (design, "qwen3"):
            if side == design:
                model = random_model(name, "bfloat16", device)
            elif side == "lekilix":
                from ..models.lekilix import lekilix_config_from_dict
                model = Model.from_random(get_architecture("Lekilix"), lekilix_config_from_dict(EQUAL_LEKILIX[name]), seed=0,
                                          dtype="bfloat16", device=device, norm_jitter=0.0)
            else:
                model = Model.from_random(get_architecture("Qwen3ForCausalLM"), qwen3_config_from_dict(EQUAL_QWEN3[name]), seed=0,
                                          dtype="bfloat16", device=device, norm_jitter=0.0)
            res = decode_and_prefill_points(model, batches, prompt_len, steps, warmup, prefill_tokens, prompt_len + 512, peaks,
                                            cuda_graphs=cuda_graphs)
            eng = res.pop("engine")
            eng.runner.check_device_status()
            row[side] = {"weight_gb": model.weight_bytes / 1e9,
                         "decode": {str(b): {k: r[k] for k in ("tokens_per_s", "ms_per_step", "roofline_frac", "launches")}
                                    for b, r in res["decode"].items()},
                         "prefill": {str(t): {k: r[k] for k in ("tokens_per_s", "ms", "tflops", "frac")} for t, r in res["prefill"].items()}}
            del eng, res, model
            gc.collect()
            torch.cuda.empty_cache()
        out[name] = row
    return out
