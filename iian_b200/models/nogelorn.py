"""Nogelorn: typed configuration, layer description and tensor names.

A decoder-only model whose layers put a norm before AND after each sub-layer: ``x += n1b(mixer(n1 x))``,
``x += n2b(ff(n2 x))`` (``iian_b200/parts/block.py: sandwich_residual``); every norm is an RMS norm whose stored weight sits
around zero (``weight_offset`` 1).  ``config.json`` lists the layers one by one (``layers``: ``type`` names the mixer,
``mixer`` its sizes, ``mlp`` the feed-forward or null) besides a few model-wide values (``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``loop``).  Per layer:

* mixer ``attention``: rotated attention over K/V heads with a sliding window that keeps the first ``mask.keep_first`` keys, a
  sink in the softmax and one sigmoid gate per head; frequencies rescaled by a ramp over the pair index with a magnitude on
  cos and sin (``iian_b200/parts/window_attention.py``, ``parts/position.py: scaled_rotary``);
* mixer ``lightning``: linear attention with one constant decay per head, silu on q, k and v, one norm over all heads and a
  sigmoid gate (``iian_b200/parts/linear_attention.py``);
* mixer ``parallel``: two mixers side by side on the same input (``iian_b200/parts/side_by_side.py``), their outputs added
  with the factors ``left_scale`` / ``right_scale`` -- left a sliding-window attention whose rotated q and k are divided by
  their root mean square per head, frequencies rescaled by wavelength bands; right linear attention with a learned decay per
  key channel (``sigmoid(.)^(1/tau)`` behind a low-rank pair of matrices whose inner size the tensor ``right.a1`` gives), a
  norm per head and a silu gate;
* feed-forward ``moe``: routed experts weighed by the softmax over the chosen (biased) router logits, plus an expert every
  token uses (``iian_b200/parts/experts.py``).

``loop`` makes the layers ``start .. stop - 1`` run ``times`` times in a row with the same weights; every run has caches and
states of its own (the run order names a layer several times, each call with its own cache id), and every run but the first
begins with ``x <- x + e``, ``e`` being what the embedding left (``iian_b200/parts/stream.py: add_embedding``).  The embedding
is multiplied by ``embedding.scale``; the output is the model's norm and the embedding table itself as the head (no scale).
Positions have no stated limit.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .galodra import _get
from .lekilix import LoopConfig
from .qwen3 import ConfigError

MAX_POSITION = 1 << 24          # the design states no limit; angles are float64 products


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[Tuple[str, float], ...]]      # the file's numbers, sorted by key; None: plain frequencies


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]
    window: Optional[int]          # keys visible to a query, itself included; None: all
    keep_first: int                # first keys that stay visible behind the window


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ChannelDecayConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class SideBySideConfig:
    left: WindowAttentionConfig
    right: ChannelDecayConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class NogelornFeedForwardConfig:
    kind: str                      # "moe" | "dense"
    ff: int                        # of one expert for "moe"
    experts: int = 0
    top: int = 0
    shared_ff: int = 0             # 0: no expert that every token uses


@dataclass(frozen=True)
class NogelornLayerConfig:
    type: str                      # "attention" | "lightning" | "parallel"
    mixer: object
    mlp: Optional[NogelornFeedForwardConfig]


@dataclass(frozen=True)
class NogelornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[NogelornLayerConfig, ...]
    loop: Optional[LoopConfig] = None
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether a run of the looped stretch other than the first starts here) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(n))
        lp = self.loop
        order = [(i, False) for i in range(lp.start)]
        for r in range(lp.times):
            order += [(i, r > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        order += [(i, False) for i in range(lp.stop, n)]
        return tuple(order)


def _rotation_from_dict(raw: Optional[Mapping[str, Any]], dim: int, where: str, keys: Tuple[str, ...]) -> Optional[RotationConfig]:
    if raw is None:
        return None
    dims = _get(raw, "dims", int, where)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where} dims must be even and at most dim ({dim}), got {dims}")
    scaling = None
    if raw.get("scaling") is not None:
        sc = _get(raw, "scaling", dict, where)
        scaling = tuple((k, _get(sc, k, float, where + " scaling")) for k in sorted(keys))
        if dict(scaling)["factor"] <= 0:
            raise ConfigError(f"config.json: {where} scaling factor must be positive")
    return RotationConfig(dims, _get(raw, "base", float, where), scaling)


def _window_attention_from_dict(raw: Mapping[str, Any], where: str, scaling_keys: Tuple[str, ...]) -> WindowAttentionConfig:
    heads, kv_heads = _get(raw, "heads", int, where), _get(raw, "kv_heads", int, where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where} has {heads} heads for {kv_heads} key/value heads")
    dim = _get(raw, "dim", int, where)
    mask = raw.get("mask")
    window, keep = None, 0
    if mask is not None:
        window = _get(mask, "size", int, where + " mask", optional=True)
        kf = mask.get("keep_first") if isinstance(mask, Mapping) else None
        if kf is not None:
            if isinstance(kf, bool) or not isinstance(kf, int) or kf < 0:
                raise ConfigError(f"config.json: {where} mask keep_first must be a non-negative integer, got {kf!r}")
            keep = kf if window is not None else 0
    return WindowAttentionConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_get(raw, "vdim", int, where),
                                 scale=_get(raw, "scale", float, where),
                                 rot=_rotation_from_dict(raw.get("rot"), dim, where + " rot", scaling_keys), window=window,
                                 keep_first=keep)


BAND_KEYS = ("factor", "low", "high", "original")
RAMP_KEYS = ("factor", "original", "fast", "slow")


def _mixer_from_dict(kind: str, raw: Mapping[str, Any], where: str):
    if kind == "attention":
        return _window_attention_from_dict(raw, where, RAMP_KEYS)
    if kind == "lightning":
        heads = _get(raw, "heads", int, where)
        decay = raw.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"config.json: {where} 'decay' must list one number per head ({heads})")
        return LightningConfig(heads=heads, dim=_get(raw, "dim", int, where), vdim=_get(raw, "vdim", int, where),
                               decay=tuple(float(d) for d in decay))
    if kind == "parallel":
        right = _get(raw, "right", dict, where)
        rw = where + " right"
        tau = _get(right, "tau", float, rw)
        if tau <= 0:
            raise ConfigError(f"config.json: {rw} tau must be positive, got {tau}")
        rank = right.get("decay_rank")
        if isinstance(rank, bool) or not isinstance(rank, int) or rank <= 0:
            raise ConfigError(f"config.json: {rw} lacks the inner size of the decay's matrices (the rows of the tensor right.a1 give it)")
        return SideBySideConfig(
            left=_window_attention_from_dict(_get(raw, "left", dict, where), where + " left", BAND_KEYS),
            right=ChannelDecayConfig(heads=_get(right, "heads", int, rw), dim=_get(right, "dim", int, rw),
                                     vdim=_get(right, "vdim", int, rw), tau=tau, rank=rank),
            left_scale=_get(raw, "left_scale", float, where), right_scale=_get(raw, "right_scale", float, where))
    raise ConfigError(f"config.json: {where} has unknown type {kind!r} (attention, lightning, parallel)")


def _mlp_from_dict(raw: Optional[Mapping[str, Any]], where: str) -> Optional[NogelornFeedForwardConfig]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, Mapping) else None
    if kind == "dense":
        return NogelornFeedForwardConfig("dense", _get(raw, "ff", int, where))
    if kind == "moe":
        expert = _get(raw, "expert", dict, where)
        router = _get(raw, "router", dict, where)
        experts, top = _get(router, "experts", int, where + " router"), _get(router, "top", int, where + " router")
        if top > experts:
            raise ConfigError(f"config.json: {where} router takes {top} of {experts} experts")
        shared = raw.get("shared")
        return NogelornFeedForwardConfig("moe", _get(expert, "ff", int, where + " expert"), experts, top,
                                         _get(shared, "ff", int, where + " shared") if shared is not None else 0)
    raise ConfigError(f"config.json: {where} has unknown kind {kind!r} (moe, dense)")


def nogelorn_config_from_dict(raw: Mapping[str, Any]) -> NogelornConfig:
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, lr in enumerate(layers_raw):
        where = f"layer {i}"
        kind = lr.get("type") if isinstance(lr, Mapping) else None
        mixer_raw = _get(lr, "mixer", dict, where) if isinstance(lr, Mapping) else None
        layers.append(NogelornLayerConfig(kind, _mixer_from_dict(kind, mixer_raw, where + " mixer"),
                                          _mlp_from_dict(lr.get("mlp"), where + " mlp")))
    norm = _get(raw, "norm", dict, "the model")
    emb = raw.get("embedding")
    scale = _get(emb, "scale", float, "embedding") if emb is not None else 1.0
    loop = None
    if raw.get("loop") is not None:
        lr = _get(raw, "loop", dict, "the model")
        start, stop, times = lr.get("start"), lr.get("stop"), lr.get("times")
        for name, v in (("start", start), ("stop", stop), ("times", times)):
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError(f"config.json: loop '{name}' must be a non-negative integer, got {v!r}")
        if not start < stop <= len(layers) or times < 1:
            raise ConfigError(f"config.json: loop runs layers {start} .. {stop} - 1 {times} times; the model has {len(layers)} layers")
        loop = LoopConfig(start, stop, times)
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
    return NogelornConfig(vocab=_get(raw, "vocab", int, "the model"), width=_get(raw, "width", int, "the model"),
                          norm_eps=_get(norm, "eps", float, "norm"), embedding_scale=scale, layers=tuple(layers), loop=loop,
                          eos_token_ids=eos_ids)


def _rotation_to_dict(r: RotationConfig) -> Dict[str, Any]:
    d: Dict[str, Any] = {"dims": r.dims, "base": r.base}
    if r.scaling is not None:
        d["scaling"] = dict(r.scaling)
    return d


def _window_attention_to_dict(m: WindowAttentionConfig) -> Dict[str, Any]:
    d: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
    if m.rot is not None:
        d["rot"] = _rotation_to_dict(m.rot)
    if m.window is not None:
        d["mask"] = {"size": m.window}
        if m.keep_first:
            d["mask"]["keep_first"] = m.keep_first
    return d


@register_architecture
class Nogelorn(Architecture):
    name = "Nogelorn"
    reads_tensor_shapes = True

    def with_tensor_sizes(self, raw: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
        """``raw`` completed with the one size that only the weight file gives: the inner size of the decay's two matrices in
        the right member of a ``parallel`` mixer, the rows of ``l<i>.mix.right.a1``.  A key that ``raw`` states stays."""
        out = copy.deepcopy(dict(raw))
        layers = out.get("layers")
        if not isinstance(layers, list):
            return out
        for i, lr in enumerate(layers):
            if not isinstance(lr, dict) or lr.get("type") != "parallel" or not isinstance(lr.get("mixer"), dict):
                continue
            right = lr["mixer"].get("right")
            shape = shapes.get(f"l{i}.mix.right.a1")
            if isinstance(right, dict) and right.get("decay_rank") is None and shape is not None and len(shape) == 2:
                right["decay_rank"] = int(shape[0])
        return out

    def load_config(self, raw: Mapping[str, Any]) -> NogelornConfig:
        return nogelorn_config_from_dict(raw)

    def config_to_dict(self, c: NogelornConfig) -> Dict[str, Any]:
        layers = []
        for lc in c.layers:
            m = lc.mixer
            if lc.type == "attention":
                mixer: Dict[str, Any] = _window_attention_to_dict(m)
            elif lc.type == "lightning":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            else:
                mixer = {"left": _window_attention_to_dict(m.left),
                         "right": {"heads": m.right.heads, "dim": m.right.dim, "vdim": m.right.vdim, "tau": m.right.tau,
                                   "decay_rank": m.right.rank},
                         "left_scale": m.left_scale, "right_scale": m.right_scale}
            if lc.mlp is None:
                mlp = None
            elif lc.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": lc.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": lc.mlp.ff}, "router": {"experts": lc.mlp.experts, "top": lc.mlp.top}}
                if lc.mlp.shared_ff:
                    mlp["shared"] = {"ff": lc.mlp.shared_ff}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.name, "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                             "embedding": {"scale": c.embedding_scale}, "layers": layers}
        if c.loop is not None:
            d["loop"] = {"start": c.loop.start, "stop": c.loop.stop, "times": c.loop.times}
        if c.eos_token_ids:
            d["eos_token_id"] = list(c.eos_token_ids)
        return d

    @staticmethod
    def _position(rot: Optional[RotationConfig], kind: str) -> PartSpec:
        if rot is None or not rot.dims:
            return PartSpec("none")
        if rot.scaling is None:
            return PartSpec("rotary", {"dim": rot.dims, "base": rot.base, "style": "neox", "max_position": MAX_POSITION})
        return PartSpec("scaled_rotary", {"dim": rot.dims, "base": rot.base, "style": "neox", "max_position": MAX_POSITION,
                                          "scaling": dict(rot.scaling, kind=kind)})

    def _window_attention(self, c: NogelornConfig, m: WindowAttentionConfig, *, scaling: str, unit_norm: bool, sink: bool,
                          head_gate: bool) -> PartSpec:
        return PartSpec("window_attention", {
            "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
            "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "sink": sink, "head_gate": head_gate,
            "unit_norm": unit_norm, "unit_norm_eps": c.norm_eps, "position": self._position(m.rot, scaling)})

    def build_spec(self, c: NogelornConfig) -> ModelSpec:
        def norm() -> PartSpec:
            return PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "weight_offset": 1.0})

        layers = []
        for lc in c.layers:
            m = lc.mixer
            if lc.type == "attention":
                mixer = self._window_attention(c, m, scaling="ramp", unit_norm=False, sink=True, head_gate=True)
            elif lc.type == "lightning":
                mixer = PartSpec("decay_linear_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "dim": m.dim, "v_dim": m.vdim, "activation": "silu",
                    "q_scale": 1.0, "decay": "head", "head_decay": m.decay, "norm": "all", "norm_eps": c.norm_eps,
                    "gate_act": "sigmoid"})
            else:
                left = self._window_attention(c, m.left, scaling="bands", unit_norm=True, sink=False, head_gate=False)
                r = m.right
                right = PartSpec("decay_linear_attention", {
                    "hidden_size": c.width, "num_heads": r.heads, "dim": r.dim, "v_dim": r.vdim, "activation": None,
                    "q_scale": r.dim ** -0.5, "decay": "channel", "decay_rank": r.rank, "tau": r.tau, "norm": "head",
                    "norm_eps": c.norm_eps, "gate_act": "silu"})
                mixer = PartSpec("side_by_side", {"hidden_size": c.width, "left": left, "right": right,
                                                  "left_scale": m.left_scale, "right_scale": m.right_scale})
            ffn, extra = None, [("mixer_post_norm", norm())]
            if lc.mlp is not None:
                if lc.mlp.kind == "dense":
                    ffn = PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": lc.mlp.ff, "activation": "silu",
                                                 "names": ("gate", "up", "down")})
                else:
                    ffn = PartSpec("routed_experts", {"hidden_size": c.width, "num_experts": lc.mlp.experts, "top": lc.mlp.top,
                                                      "intermediate_size": lc.mlp.ff, "activation": "silu", "score": "softmax_top",
                                                      "weight_on": "output", "shared_intermediate_size": lc.mlp.shared_ff})
                extra.append(("feed_forward_post_norm", norm()))
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm(),
                                    feed_forward_norm=norm() if ffn is not None else None, arrangement="sandwich_residual",
                                    extra=tuple(extra)))
        again = any(starts for _, starts in c.run_order())
        stream_parts = (PartSpec("add_embedding", {}),) if again else ()
        order = tuple(LayerCall(layer=i, cache=idx, before=0 if starts else None)
                      for idx, (i, starts) in enumerate(c.run_order()))           # every run of a layer has a cache of its own
        return ModelSpec(
            hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": c.embedding_scale}),
            layers=tuple(layers), order=order, final_norm=norm(),
            head=PartSpec("lm_head", {"hidden_size": c.width, "vocab_size": c.vocab, "tied": True}),
            stream_parts=stream_parts)

    SLOTS = {"mixer_norm": "norm1", "mixer_post_norm": "norm1b", "feed_forward_norm": "norm2", "feed_forward_post_norm": "norm2b"}

    def tensor_name(self, scope: tuple, local: str) -> str:
        if scope[0] == "embedding":
            return "embed"
        if scope[0] == "final_norm":
            return "final.norm"
        if scope[0] == "layer":
            i, slot = scope[1], scope[2]
            if slot == "mixer":
                return f"l{i}.mix.{local}"
            if slot == "feed_forward":
                return f"l{i}.mlp.{local}"
            if slot in self.SLOTS:
                return f"l{i}.{self.SLOTS[slot]}"
        raise KeyError(scope)
