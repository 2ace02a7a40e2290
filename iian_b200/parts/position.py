"""Position encodings.

``rotary``: rotation of pairs of the head by angles ``pos * base^(-2j/dim)``
(third_party/ggml/src/ggml-cpu/ops.cpp:5958-5990; pairing styles :6063-6079).  The part owns the
float32 table of ``base^(-2j/dim)``; the attention mixer hands it to the fused kernel, which
multiplies by the position and takes sin/cos in float32.  ``dim`` may be smaller than the head
(partial rotation); Qwen3 rotates the whole head (src/iian/arch/qwen3.cpp:66).

``scaled_rotary``: the same rotation with frequencies rescaled for contexts longer than the ones the model first saw, in one
of two ways (``scaling["kind"]``), and optionally a magnitude on cos and sin.  Its table is made with the angle and the
functions in float64 (``table64``); only mixers that read ``table64`` can use it.

``none``: no position signal (the mixer stores K unrotated).

Another encoding is another class registered with ``register_position``.  If it cannot be expressed
as a rotation table it sets ``fused = False`` and implements ``apply(q, k, positions, ctx)``, which the
attention mixer calls on the projected heads before they are stored.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position

ROPE_STYLES = {"neox": 0, "interleaved": 1}


@register_position("rotary")
class Rotary(PositionEncoding):
    """params: ``dim`` (rotated dims, even), ``base``, ``style`` (``neox`` pairs (j, j+dim/2),
    ``interleaved`` pairs (2j, 2j+1)), ``max_position``; optional ``frequency_scale`` (linear scaling,
    the reference's ``freq_scale``, default 1)."""

    fused = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.dim = int(spec["dim"])
        if self.dim <= 0 or self.dim % 2:
            raise ValueError(f"rotary: dim must be positive and even, got {self.dim}")
        self.base = float(spec["base"])
        style = spec.params.get("style", "neox")
        if style not in ROPE_STYLES:
            raise ValueError(f"rotary: unknown style '{style}' ({', '.join(ROPE_STYLES)})")
        self.style = ROPE_STYLES[style]
        self.max_position = int(spec.params.get("max_position", 0))
        scale = float(spec.params.get("frequency_scale", 1.0))
        j = torch.arange(self.dim // 2, dtype=torch.float64)
        inv = scale * torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * j / self.dim)
        self.inv_freq = inv.to(torch.float32).to(device)
        self.inv_freq64 = inv.to(device)         # for kernels that form the angle in float64
        self.key = ("rotary", self.dim, self.base, scale)

    def table(self, ctx):
        """cos and sin of this step's angles, float32 [N, dim / 2, 2].  The angles depend on the positions
        and on this part's constants only, so one table per step serves every layer that rotates alike."""
        from .. import ops
        tables = ctx.step_cache.setdefault("rotary_tables", {}) if hasattr(ctx, "step_cache") else {}
        t = tables.get(self.key)
        if t is None:
            k = ops.kernels()
            if not hasattr(k, "rotary_table"):
                return None
            n = ctx.positions.shape[0]
            t = ctx.buf(f"rotary_table_{len(tables)}", (n, self.dim // 2, 2), torch.float32)
            k.rotary_table(self.inv_freq, ctx.positions, self.dim // 2, t)
            tables[self.key] = t
        return t


    def table64(self, ctx):
        """cos and sin of this step's angles times ``magnitude``, float32 [N, dim / 2, 2], with the product ``position *
        frequency`` and the functions in float64: exact at any position.  One table per step serves every layer that rotates
        alike."""
        from .. import ops
        tables = ctx.step_cache.setdefault("rotary_tables64", {})
        t = tables.get(self.key)
        if t is None:
            n = ctx.positions.shape[0]
            t = ctx.buf(f"rotary_table64_{len(tables)}", (n, self.dim // 2, 2), torch.float32)
            ops.kernels().rotary_table_scaled(self.inv_freq64, ctx.positions, self.dim // 2, self.magnitude, t)
            tables[self.key] = t
        return t

    magnitude = 1.0


def banded_frequencies(inv: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Rescaling by wavelength bands.  With ``l = 2 pi / f``: ``f`` stays where ``l < original / high``, becomes ``f / factor``
    where ``l > original / low``, and between the two is ``(1 - s) f / factor + s f`` with ``s = (original / l - low) /
    (high - low)``.  float64 in and out."""
    wave = 2.0 * math.pi / inv
    s = (original / wave - low) / (high - low)
    mid = (1.0 - s) * inv / factor + s * inv
    return torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, mid))


def ramped_frequencies(inv: torch.Tensor, dim: int, base: float, factor: float, original: float, fast: float, slow: float):
    """Rescaling by a ramp over the pair index i.  With ``c(t) = dim ln(original / (2 pi t)) / (2 ln base)``, ``lo =
    max(floor(c(fast)), 0)``, ``hi = min(ceil(c(slow)), dim - 1)`` and ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``
    the frequency is ``r_i f_i / factor + (1 - r_i) f_i``; cos and sin are multiplied by ``0.1 ln(factor) + 1``.  Returns
    ``(frequencies float64, magnitude)``."""
    def c(turns: float) -> float:
        return dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(c(fast)), 0)
    hi = min(math.ceil(c(slow)), dim - 1)
    i = torch.arange(dim // 2, dtype=torch.float64)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / factor * r + inv * (1.0 - r), 0.1 * math.log(factor) + 1.0


@register_position("scaled_rotary")
class ScaledRotary(Rotary):
    """params: those of ``rotary`` (``frequency_scale`` excluded) and ``scaling``: a mapping with ``kind`` = ``bands``
    (``factor``, ``low``, ``high``, ``original``) or ``ramp`` (``factor``, ``original``, ``fast``, ``slow``)."""

    fused = False          # the kernels that take a rotation's float32 frequencies know nothing of a magnitude

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        sc = dict(spec["scaling"])
        kind = sc.get("kind")
        j = torch.arange(self.dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * j / self.dim)
        if kind == "bands":
            inv = banded_frequencies(inv, float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
        elif kind == "ramp":
            inv, self.magnitude = ramped_frequencies(inv, self.dim, self.base, float(sc["factor"]), float(sc["original"]),
                                                     float(sc["fast"]), float(sc["slow"]))
        else:
            raise ValueError(f"scaled_rotary: unknown kind of scaling '{kind}' (bands, ramp)")
        self.inv_freq = inv.to(torch.float32).to(device)
        self.inv_freq64 = inv.to(device)
        self.key = ("scaled_rotary", self.dim, self.base, kind, tuple(sorted((k, float(v)) for k, v in sc.items() if k != "kind")))

    def table(self, ctx):
        raise NotImplementedError("scaled_rotary: only mixers that read table64 (angles in float64, with the magnitude) can use it")

    def apply(self, qkv, num_heads, num_kv_heads, head_dim, ctx):
        raise NotImplementedError("scaled_rotary: this mixer's kernels take plain rotations only")


@register_position("none")
class NoPosition(PositionEncoding):
    fused = True
    dim = 0
    style = 0
    inv_freq = None
    inv_freq64 = None
