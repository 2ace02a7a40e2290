"""Senadra: typed configuration, layer description and tensor names.

A decoder-only model of pre-norm layers whose sub-layer outputs enter the stream with a factor:
``x += m mixer(norm1 x)``, ``x += m ff(norm2 x)``, then a second per-token input ``x += m unit_rms(P (gelu(G x) * e)) * w``
with ``e`` the layer's slice of a second embedding table (``iian_b200/parts/block.py: scaled_residual``).  ``config.json``
lists the layers one by one (``layers``: ``type`` names the mixer, ``mixer`` its sizes, ``mlp`` the feed-forward or null)
besides a few model-wide values (``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``token_side.dim``,
``logit_softcap``).  Per layer:

* mixer ``attention``: attention without rotation whose values have a size of their own and are cached divided by their
  root mean square, visible keys limited to the query's chunk of positions, a penalty ``r1 ln(1 + r2 distance)`` on the
  score, a sigmoid gate on the output; with ``kv_from`` = j the layer has no key / value projections and reads the cache
  layer j fills (``iian_b200/parts/chunked_attention.py``);
* mixer ``latent_attention``: attention over a cached low-rank latent with a shared rotated key part (interleaved pairs),
  queries through a normalised latent of their own, a sigmoid gate on the output (``iian_b200/parts/latent_attention.py``);
* mixer ``channel_delta``: the gated delta rule with a decay per key channel, short convolutions in front, a state per
  request (``iian_b200/parts/delta_rule.py``).  The inner sizes of its two low-rank maps are not in ``config.json``: the
  shapes of the tensors ``a1`` and ``g1`` give them (``with_tensor_sizes``), unless the keys ``decay_rank`` /
  ``gate_rank`` state them;
* feed-forward ``dense``: no gate, the xIELU activation with two learned numbers (``iian_b200/parts/mlp.py: plain_mlp``).

The output is the model's RMS norm, an untied head and ``c tanh(logits / c)``.  Positions have no stated limit.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .galodra import FeedForwardConfig, _get
from .qwen3 import ConfigError

MAX_POSITION = 1 << 24          # the design states no limit; angles are float64 products


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]           # positions per chunk; None: every earlier key is visible
    kv_from: Optional[int]         # the layer whose keys and values this one reads; None: its own


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: Optional[int]          # None: the queries are projected directly
    scale: float
    rot_dims: int                  # how many of the rot_dim entries rotate (0: none)
    rot_base: float


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class SenadraLayerConfig:
    type: str                      # "attention" | "latent_attention" | "channel_delta"
    mixer: object
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class SenadraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    side_dim: int                  # 0: no second per-token input
    layers: Tuple[SenadraLayerConfig, ...]
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


def _attention_from_dict(raw: Mapping[str, Any], where: str, index: int) -> ChunkedAttentionConfig:
    heads, kv_heads = _get(raw, "heads", int, where), _get(raw, "kv_heads", int, where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where} has {heads} heads for {kv_heads} key/value heads")
    mask = raw.get("mask")
    chunk = _get(mask, "size", int, where + " mask", optional=True) if mask is not None else None
    src = raw.get("kv_from")
    if src is not None and (isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index):
        raise ConfigError(f"config.json: {where} 'kv_from' must name an earlier layer, got {src!r}")
    return ChunkedAttentionConfig(heads=heads, kv_heads=kv_heads, dim=_get(raw, "dim", int, where), vdim=_get(raw, "vdim", int, where),
                                  scale=_get(raw, "scale", float, where), chunk=chunk, kv_from=src)


def _latent_from_dict(raw: Mapping[str, Any], where: str) -> LatentConfig:
    rot = raw.get("rot")
    rot_dim = _get(raw, "rot_dim", int, where)
    rot_dims, base = 0, 10000.0
    if rot is not None:
        rot_dims = _get(rot, "dims", int, where + " rot")
        base = _get(rot, "base", float, where + " rot")
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"config.json: {where} rot.dims must be even and at most rot_dim ({rot_dim}), got {rot_dims}")
    return LatentConfig(heads=_get(raw, "heads", int, where), dim=_get(raw, "dim", int, where), rot_dim=rot_dim,
                        vdim=_get(raw, "vdim", int, where), kv_rank=_get(raw, "kv_rank", int, where),
                        q_rank=_get(raw, "q_rank", int, where, optional=True), scale=_get(raw, "scale", float, where),
                        rot_dims=rot_dims, rot_base=base)


def _delta_from_dict(raw: Mapping[str, Any], where: str) -> DeltaConfig:
    heads, kv_heads = _get(raw, "heads", int, where), _get(raw, "kv_heads", int, where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where} has {heads} heads for {kv_heads} query/key heads")
    ranks = []
    for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
        r = _get(raw, key, int, where, optional=True)
        if r is None:
            raise ConfigError(f"config.json: {where} does not state '{key}', and no weight file is at hand whose tensor "
                              f"'{tensor}' would give it")
        ranks.append(r)
    return DeltaConfig(heads=heads, kv_heads=kv_heads, dim=_get(raw, "dim", int, where), vdim=_get(raw, "vdim", int, where),
                       conv=_get(raw, "conv", int, where), decay_rank=ranks[0], gate_rank=ranks[1])


def _mlp_from_dict(raw: Optional[Mapping[str, Any]], where: str) -> Optional[FeedForwardConfig]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, Mapping) else None
    if kind == "dense":
        return FeedForwardConfig("dense", _get(raw, "ff", int, where))
    raise ConfigError(f"config.json: {where} has unknown kind {kind!r} (dense)")


def senadra_config_from_dict(raw: Mapping[str, Any]) -> SenadraConfig:
    layers_raw = raw.get("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, lr in enumerate(layers_raw):
        where = f"layer {i}"
        kind = lr.get("type") if isinstance(lr, Mapping) else None
        mixer_raw = _get(lr, "mixer", dict, where) if isinstance(lr, Mapping) else None
        if kind == "attention":
            mixer: object = _attention_from_dict(mixer_raw, where + " mixer", i)
        elif kind == "latent_attention":
            mixer = _latent_from_dict(mixer_raw, where + " mixer")
        elif kind == "channel_delta":
            mixer = _delta_from_dict(mixer_raw, where + " mixer")
        else:
            raise ConfigError(f"config.json: {where} has unknown type {kind!r} (attention, latent_attention, channel_delta)")
        layers.append(SenadraLayerConfig(kind, mixer, _mlp_from_dict(lr.get("mlp"), where + " mlp")))
    for i, lc in enumerate(layers):
        if lc.type == "attention" and lc.mixer.kv_from is not None:
            src = layers[lc.mixer.kv_from]
            m, s = lc.mixer, src.mixer
            if src.type != "attention" or s.kv_from is not None:
                raise ConfigError(f"config.json: layer {i} reads the keys and values of layer {m.kv_from}, which projects none")
            if (s.kv_heads, s.dim, s.vdim) != (m.kv_heads, m.dim, m.vdim):
                raise ConfigError(f"config.json: layer {i} reads the keys and values of layer {m.kv_from}, whose heads differ")
    norm = _get(raw, "norm", dict, "the model")
    side = raw.get("token_side")
    side_dim = _get(side, "dim", int, "token_side") if side is not None else 0
    cap = _get(raw, "logit_softcap", float, "the model", optional=True)
    if cap is not None and cap <= 0:
        raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
    mult = _get(raw, "residual_mult", float, "the model", optional=True)
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
    return SenadraConfig(vocab=_get(raw, "vocab", int, "the model"), width=_get(raw, "width", int, "the model"),
                         norm_eps=_get(norm, "eps", float, "norm"), residual_mult=1.0 if mult is None else mult,
                         logit_softcap=cap, side_dim=side_dim, layers=tuple(layers), eos_token_ids=eos_ids)


@register_architecture
class Senadra(Architecture):
    name = "Senadra"
    reads_tensor_shapes = True

    def with_tensor_sizes(self, raw: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
        """``raw`` completed with the sizes that only the weight file's tensors give: the inner sizes of a delta-rule mixer's
        two low-rank maps, the rows of ``l<i>.mix.a1`` and ``l<i>.mix.g1``.  Keys that ``raw`` states stay as they are."""
        out = copy.deepcopy(dict(raw))
        layers = out.get("layers")
        if not isinstance(layers, list):
            return out
        for i, lr in enumerate(layers):
            if not isinstance(lr, dict) or lr.get("type") != "channel_delta" or not isinstance(lr.get("mixer"), dict):
                continue
            for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                shape = shapes.get(f"l{i}.mix.{tensor}")
                if lr["mixer"].get(key) is None and shape is not None and len(shape) == 2:
                    lr["mixer"][key] = int(shape[0])
        return out

    def load_config(self, raw: Mapping[str, Any]) -> SenadraConfig:
        return senadra_config_from_dict(raw)

    def config_to_dict(self, c: SenadraConfig) -> Dict[str, Any]:
        layers = []
        for lc in c.layers:
            m = lc.mixer
            if lc.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            elif lc.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
                if m.q_rank is not None:
                    mixer["q_rank"] = m.q_rank
                if m.rot_dims:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv,
                         "decay_rank": m.decay_rank, "gate_rank": m.gate_rank}
            mlp = None if lc.mlp is None else {"kind": "dense", "ff": lc.mlp.ff}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.name, "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                             "residual_mult": c.residual_mult, "layers": layers}
        if c.side_dim:
            d["token_side"] = {"dim": c.side_dim}
        if c.logit_softcap is not None:
            d["logit_softcap"] = c.logit_softcap
        if c.eos_token_ids:
            d["eos_token_id"] = list(c.eos_token_ids)
        return d

    def build_spec(self, c: SenadraConfig) -> ModelSpec:
        def norm() -> PartSpec:
            return PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps})

        layers = []
        for i, lc in enumerate(c.layers):
            m = lc.mixer
            if lc.type == "attention":
                mixer = PartSpec("chunked_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
                    "scale": m.scale, "chunk": m.chunk, "window": None, "value_norm": True, "value_norm_eps": c.norm_eps,
                    "distance_penalty": True, "output_gate": True, "owns_kv": m.kv_from is None})
            elif lc.type == "latent_attention":
                position = (PartSpec("rotary", {"dim": m.rot_dims, "base": m.rot_base, "style": "interleaved",
                                                "max_position": MAX_POSITION}) if m.rot_dims else PartSpec("none"))
                mixer = PartSpec("latent_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
                    "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": c.norm_eps, "window": None,
                    "sink": False, "output_gate": True, "position": position})
            else:
                mixer = PartSpec("gated_delta_rule", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim, "v_dim": m.vdim,
                    "conv": m.conv, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank, "norm_eps": c.norm_eps})
            ffn = None
            if lc.mlp is not None:
                ffn = PartSpec("plain_mlp", {"hidden_size": c.width, "intermediate_size": lc.mlp.ff, "activation": "xielu",
                                             "names": ("up", "down", "act")})
            extra = [("residual_mult", PartSpec("constant", {"value": c.residual_mult}))]
            if c.side_dim:
                extra.append(("token_side", PartSpec("token_side", {"hidden_size": c.width, "dim": c.side_dim,
                                                                    "offset": i * c.side_dim, "eps": c.norm_eps})))
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm(),
                                    feed_forward_norm=norm() if ffn is not None else None,
                                    arrangement="scaled_residual", extra=tuple(extra)))
        # a layer that reads another's keys and values works on that layer's cache and writes nothing
        order = tuple(LayerCall(layer=i, cache=i if getattr(lc.mixer, "kv_from", None) is None else lc.mixer.kv_from,
                                writes_cache=getattr(lc.mixer, "kv_from", None) is None)
                      for i, lc in enumerate(c.layers))
        return ModelSpec(
            hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width,
                                                   "side_width": c.side_dim * len(c.layers)}),
            layers=tuple(layers), order=order, final_norm=norm(),
            head=PartSpec("lm_head", {"hidden_size": c.width, "vocab_size": c.vocab, "tied": False,
                                      "softcap": c.logit_softcap}))

    def tensor_name(self, scope: tuple, local: str) -> str:
        if scope[0] == "embedding":
            return "side.embed" if local == "side" else "embed"
        if scope[0] == "final_norm":
            return "final.norm"
        if scope[0] == "head":
            return "head"
        if scope[0] == "layer":
            i, slot = scope[1], scope[2]
            if slot == "mixer":
                return f"l{i}.mix.{local}"
            if slot == "feed_forward":
                return f"l{i}.mlp.{local}"
            if slot == "mixer_norm":
                return f"l{i}.norm1"
            if slot == "feed_forward_norm":
                return f"l{i}.norm2"
            if slot == "token_side":
                return f"l{i}.side.{local}"
        raise KeyError(scope)
