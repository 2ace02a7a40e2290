"""How a layer's parts are arranged.

A block implements one arrangement (``LayerSpec.arrangement``) and is registered under its name with
``register_block``.  What the model asks of a block: ``__init__(spec, dtype, device)`` builds its parts from the
slots of the ``LayerSpec`` it understands; ``parts()`` lists them with the slot names their tensors go under;
``cache_need()`` says what the cache of a call to this layer must hold (a ``KVNeed``, a ``StateNeed`` or None);
``forward(residual, delta, ctx, cache, writes_cache, select_rows)`` takes the float32 residual stream and the
not-yet-added output of whatever ran before, and returns the same pair.

``pre_norm_residual`` (src/iian/arch/qwen3.cpp:74-100): ``x += mixer(norm(x))``; ``x += ffn(norm(x))``.
The add that closes one sub-layer is fused into the norm that opens the next: a block receives the
float32 residual and the not-yet-added output of the previous sub-layer (``delta``) and returns the
same pair.

Row selection: in the last entry of the run order only the rows whose logits are wanted go on after
the mixer -- both the mixer's output and the residual (src/iian/arch/qwen3.cpp:91,
src/iian/graph.cpp:356-358) -- so the last feed-forward, the final norm and the head run on those rows.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..config.spec import LayerSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, NormOut, Prenormed, register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock:
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        missing = [s for s in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm") if spec.slot(s) is None]
        if missing:
            raise ValueError(f"arrangement pre_norm_residual needs the slots {', '.join(missing)}")
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)

    def parts(self):
        """(slot name, part) pairs; the slot name is what the architecture maps to file names."""
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward))

    def cache_need(self):
        return self.mixer.cache_need()

    accepts_next_norm = True

    @staticmethod
    def _norm_out(norm, consumer, residual: torch.Tensor, n_rows: int, name: str) -> Optional[NormOut]:
        """A request to fold ``norm`` into the products around it, if the norm allows it and ``consumer`` (the part
        that follows it) can take rows that still lack the factor per row."""
        if norm is None or consumer is None:
            return None
        fold = norm.foldable()
        if fold is None or not consumer.takes_prenormed(n_rows):
            return None
        return NormOut(residual, norm, fold[0], fold[1], name)

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool,
                select_rows: Optional[torch.Tensor], next_norm=None, next_consumer=None):
        """``delta`` is the not-yet-added output of the sub-layer before this block, or a ``Prenormed`` for this
        block's first norm (then the sum is already in ``residual``).  ``next_norm`` / ``next_consumer``: the norm
        and the part that follow this block's feed-forward, if its last product may prepare their input."""
        if isinstance(delta, Prenormed):
            if delta.norm is not self.mixer_norm:
                raise RuntimeError("block: received rows prepared for another norm")
            h = delta
        else:
            h = self.mixer_norm.forward(residual, delta, ctx)
        n_rows = residual.shape[0]
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        request = None
        if not gathers and self.mixer.folds_norm_out:
            request = self._norm_out(self.feed_forward_norm, self.feed_forward, residual, n_rows, "mixer")
        y = self.mixer.forward(h, ctx, cache, writes_cache, norm_out=request) if request is not None \
            else self.mixer.forward(h, ctx, cache, writes_cache)
        if gathers:
            k = ops.kernels()
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y = res_sel, y_sel
        h2 = y if isinstance(y, Prenormed) else self.feed_forward_norm.forward(residual, y, ctx)
        request = None
        if self.feed_forward.folds_norm_out:
            request = self._norm_out(next_norm, next_consumer, residual, residual.shape[0], "feed_forward")
        d = self.feed_forward.forward(h2, ctx, norm_out=request) if request is not None else self.feed_forward.forward(h2, ctx)
        return residual, d


@register_block("parallel_residual")
class ParallelResidualBlock:
    """``h = norm(x)``; ``x += mixer(h) + ffn(h)``: ONE norm, and both sub-layers read its output.

    Slots: ``mixer_norm`` (the layer's only norm), ``mixer``, optionally ``feed_forward`` (a layer without one adds the
    mixer's output alone).  What the block hands on as ``delta`` is the PAIR (mixer output, feed-forward output): the norm
    that comes next adds ``x + (d1 + d2)`` in float32 before it normalises, as the single-delta form does for one.
    With ``select_rows`` (the run order's last entry) the mixer sees every row (its cache or state needs them), the
    feed-forward only the selected ones."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        if spec.slot("mixer") is None or spec.slot("mixer_norm") is None:
            raise ValueError("arrangement parallel_residual needs the slots mixer, mixer_norm")
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None

    def parts(self):
        out = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer)]
        if self.feed_forward is not None:
            out.append(("feed_forward", self.feed_forward))
        return tuple(out)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool, select_rows: Optional[torch.Tensor]):
        h = self.mixer_norm.forward(residual, delta, ctx)        # residual += what was owed; h = norm(residual)
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        rows = None
        if gathers:
            k = ops.kernels()
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y = res_sel, y_sel
            if self.feed_forward is not None:
                h_sel = ctx.buf("normed_rows", (r, h.shape[1]), h.dtype)
                k.gather_rows(h, select_rows, h_sel)
                h, rows = h_sel, select_rows
        if self.feed_forward is None:
            return residual, y
        if getattr(self.feed_forward, "needs_tokens", False):
            z = self.feed_forward.forward(h, ctx, rows=rows)
        else:
            z = self.feed_forward.forward(h, ctx)
        return residual, (y, z)


class TokenSide:
    """A second input per layer that depends on the token id alone: with ``e`` the layer's slice of the token's row of a
    table shared by all layers (held by the embedding part, ``side_width`` wide), ``x`` the stream after the layer's
    sub-layers and ``m`` the residual factor,

        g = gelu_tanh(G x) * e;    y = P g;    x <- x + m * y / sqrt(mean(y^2) + eps) * w

    params: ``hidden_size``, ``dim`` (the slice's size), ``offset`` (its first column in the table), ``eps``."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.hidden = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.offset = int(spec["offset"])
        self.eps = float(spec["eps"])
        self.w_gate = self.w_proj = self.norm_w = None

    def tensors(self):
        from ..weights.loader import TensorSpec
        return {"gate": TensorSpec((self.dim, self.hidden)), "proj": TensorSpec((self.hidden, self.dim)),
                "norm": TensorSpec((self.hidden,), init="ones_jitter")}

    def bind(self, tensors) -> None:
        self.w_gate = tensors["gate"].contiguous()
        self.w_proj = tensors["proj"].contiguous()
        self.norm_w = tensors["norm"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("residual_ops", "gemm_simt")

    def forward(self, residual: torch.Tensor, x_act: torch.Tensor, mult: float, ctx, rows: Optional[torch.Tensor]) -> None:
        """Adds into ``residual`` in place.  ``x_act``: the stream in the activation dtype; ``rows``: the step's rows the
        stream's rows stand for (None: all, in order)."""
        table = ctx.step_cache.get("token_side_table")
        if table is None:
            raise RuntimeError("token_side: the embedding holds no second table (side_width)")
        k = ops.kernels()
        n = residual.shape[0]
        g = ctx.buf("side_gate", (n, self.dim), self.dtype)
        k.linear(x_act, self.w_gate, g)
        ge = ctx.buf("side_gated", (n, self.dim), self.dtype)
        k.gelu_mul_table(g, table, self.offset, ctx.tokens, rows, ge)
        y = ctx.buf("side_out", (n, self.hidden), self.dtype)
        k.linear(ge, self.w_proj, y)
        k.scaled_add_unit_rms(residual, y, mult, self.norm_w, self.eps)


@register_block("scaled_residual")
class ScaledResidualBlock:
    """``x += m mixer(norm1 x)``; ``x += m ffn(norm2 x)``; optionally ``x += m side(x, token)``: the pre-norm arrangement
    with a factor ``m`` on everything that is added to the stream.

    Slots: ``mixer_norm``, ``mixer``; optionally ``feed_forward`` with ``feed_forward_norm`` (a layer without one ends
    after the mixer's sum); in ``extra``: ``residual_mult`` as ``PartSpec("constant", {"value": m})`` and optionally
    ``token_side`` (:class:`TokenSide`).  The sum that closes a sub-layer rides in the norm kernel that opens the next
    (``x += m d`` in float32, then the norm); the block's last sum leaves the stream complete, so it hands on no addend.
    With ``select_rows`` (the run order's last entry) only the wanted rows go on after the mixer."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        if spec.slot("mixer") is None or spec.slot("mixer_norm") is None:
            raise ValueError("arrangement scaled_residual needs the slots mixer, mixer_norm")
        if (spec.slot("feed_forward") is None) != (spec.slot("feed_forward_norm") is None):
            raise ValueError("arrangement scaled_residual: feed_forward and feed_forward_norm come together")
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device) if spec.feed_forward is not None else None
        m = spec.slot("residual_mult")
        self.mult = float(m["value"]) if m is not None else 1.0
        side = spec.slot("token_side")
        self.token_side = TokenSide(side, dtype, device) if side is not None else None

    def parts(self):
        out = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer)]
        if self.feed_forward is not None:
            out += [("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward)]
        if self.token_side is not None:
            out.append(("token_side", self.token_side))
        return tuple(out)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool, select_rows: Optional[torch.Tensor]):
        k = ops.kernels()
        h = self.mixer_norm.forward(residual, delta, ctx)            # what the layer before left to add has no factor
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        rows = None
        if gathers:
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y, rows = res_sel, y_sel, select_rows
        if self.feed_forward is not None:
            h2 = self.feed_forward_norm.forward(residual, y, ctx, delta_scale=self.mult)
            y = self.feed_forward.forward(h2, ctx)
        # the block's last sum; the token side reads the finished stream
        if self.token_side is None:
            k.scaled_add_rms_norm(residual, y, self.mult, None, 0.0, None)
            return residual, None
        if self.dtype == torch.float32:
            k.scaled_add_rms_norm(residual, y, self.mult, None, 0.0, None)
            x_act = residual
        else:
            x_act = ctx.buf("stream_act", residual.shape, self.dtype)
            k.scaled_add_rms_norm(residual, y, self.mult, None, 0.0, None, copy=x_act)
        self.token_side.forward(residual, x_act, self.mult, ctx, rows)
        return residual, None


@register_block("sandwich_residual")
class SandwichResidualBlock:
    """``x += nb1(mixer(n1 x))``; ``x += nb2(ffn(n2 x))``: a norm before AND after each sub-layer.

    Slots: ``mixer_norm``, ``mixer``; optionally ``feed_forward`` with ``feed_forward_norm``; in ``extra``
    ``mixer_post_norm`` and (with a feed-forward) ``feed_forward_post_norm``, norms that offer ``as_addend`` (``rms_norm``).
    A sub-layer's output is not added by a kernel of its own: wrapped as a ``NormedAddend`` it goes to the norm that runs
    next, whose kernel normalises it, adds it to the float32 stream and normalises the stream (the block's last one is handed
    on as ``delta``).  With ``select_rows`` (the run order's last entry) only the wanted rows go on after the mixer."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        need = ["mixer", "mixer_norm", "mixer_post_norm"]
        if spec.slot("feed_forward") is not None:
            need += ["feed_forward_norm", "feed_forward_post_norm"]
        missing = [s for s in need if spec.slot(s) is None]
        if missing:
            raise ValueError(f"arrangement sandwich_residual needs the slots {', '.join(missing)}")
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.mixer_post_norm = NORMS.build(spec.slot("mixer_post_norm"), dtype, device)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)
            self.feed_forward_post_norm = NORMS.build(spec.slot("feed_forward_post_norm"), dtype, device)
        for norm in (self.mixer_post_norm, self.feed_forward_post_norm):
            if norm is not None and not hasattr(norm, "as_addend"):
                raise ValueError("arrangement sandwich_residual needs post-norms that can ride in the next norm's sum (rms_norm)")

    def parts(self):
        out = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer), ("mixer_post_norm", self.mixer_post_norm)]
        if self.feed_forward is not None:
            out += [("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward),
                    ("feed_forward_post_norm", self.feed_forward_post_norm)]
        return tuple(out)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool, select_rows: Optional[torch.Tensor]):
        h = self.mixer_norm.forward(residual, delta, ctx)            # residual += what was owed; h = n1(residual)
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        if gathers:
            k = ops.kernels()
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y = res_sel, y_sel
        owed = self.mixer_post_norm.as_addend(y)
        if self.feed_forward is None:
            return residual, owed
        h2 = self.feed_forward_norm.forward(residual, owed, ctx)
        z = self.feed_forward.forward(h2, ctx)
        return residual, self.feed_forward_post_norm.as_addend(z)


class SigmoidGate:
    """A gate of a sub-layer's output: ``sigmoid(W h + b)`` per element, ``h`` the sub-layer's input.  params: ``size``.
    The matrix rides as extra rows in the sub-layer's own first product (``stack_rows``); the bias and the sigmoid are
    applied by the kernel that adds the sub-layer's output to the stream."""

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.size = int(spec["size"])
        self.weight = self.bias = None
        self.graph_safe = True

    def tensors(self):
        from ..weights.loader import TensorSpec
        return {"weight": TensorSpec((self.size, self.size)), "bias": TensorSpec((self.size,), init="zeros")}

    def bind(self, tensors) -> None:
        self.weight = tensors["weight"]
        self.bias = tensors["bias"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("postnorm",)


class DepthMix:
    """What a layer hands on is a learned mix of the embedding output and every layer result so far:
    ``x = sum_j c[j] X_j``, ``j = 0 .. terms - 1``.  params: ``terms``."""

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.terms = int(spec["terms"])
        self.coef = None
        self.graph_safe = True

    def tensors(self):
        from ..weights.loader import TensorSpec
        return {"weight": TensorSpec((self.terms,), init="ones_jitter")}

    def bind(self, tensors) -> None:
        self.coef = tensors["weight"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("postnorm",)


@register_block("post_norm_residual")
class PostNormResidualBlock:
    """``y = norm1(alpha * x + g1(x) * mixer(x))``; ``z = norm2(alpha * y + g2(y) * ffn(y))``: the norm comes AFTER the sum,
    the sub-layers read the stream itself, and the skip path is scaled by ``alpha``.

    Slots: ``mixer``, ``mixer_norm`` (the norm after the mixer's sum), optionally ``feed_forward`` with
    ``feed_forward_norm`` (a layer without feed-forward ends after the first norm); in ``extra``, all optional:
    ``mixer_gate`` / ``feed_forward_gate`` (``sigmoid_gate``: the sub-layer's output is multiplied by
    ``sigmoid(W h + b)`` of its input before the sum) and ``depth_mix`` (the stream handed to the next layer is a learned
    mix of the embedding output and all layer results so far, ``terms`` of them).  ``extra`` also carries the constants
    ``alpha`` as ``("alpha", PartSpec("constant", {"value": a}))``.

    The norm kernel does the scaled skip, the gate's bias and sigmoid, the product with the sub-layer's output, the sum
    and the LayerNorm in one pass, and leaves the float32 stream plus its copy in the activation dtype.  The stream
    between layers is float32 in ``residual``; ``delta`` stays None (nothing is left to add)."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        if spec.slot("mixer") is None or spec.slot("mixer_norm") is None:
            raise ValueError("arrangement post_norm_residual needs the slots mixer, mixer_norm")
        if (spec.slot("feed_forward") is None) != (spec.slot("feed_forward_norm") is None):
            raise ValueError("arrangement post_norm_residual: feed_forward and feed_forward_norm come together")
        self.spec = spec
        self.dtype = dtype
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device) if spec.feed_forward is not None else None
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "sum_norm"):
                raise ValueError("arrangement post_norm_residual needs norms that fuse the sum (layer_norm)")
        alpha = spec.slot("alpha")
        self.alpha = float(alpha["value"]) if alpha is not None else 1.0
        g1, g2, mix = spec.slot("mixer_gate"), spec.slot("feed_forward_gate"), spec.slot("depth_mix")
        self.mixer_gate = SigmoidGate(g1, dtype, device) if g1 is not None else None
        self.feed_forward_gate = SigmoidGate(g2, dtype, device) if g2 is not None and self.feed_forward is not None else None
        self.depth_mix = DepthMix(mix, dtype, device) if mix is not None else None
        self._stacked = False

    def parts(self):
        out = [("mixer", self.mixer), ("mixer_norm", self.mixer_norm)]
        if self.feed_forward is not None:
            out += [("feed_forward", self.feed_forward), ("feed_forward_norm", self.feed_forward_norm)]
        for name in ("mixer_gate", "feed_forward_gate", "depth_mix"):
            if getattr(self, name) is not None:
                out.append((name, getattr(self, name)))
        return tuple(out)

    def cache_need(self):
        return self.mixer.cache_need()

    def _stack_gates(self) -> None:
        """After the weights are bound: put each gate's matrix under its sub-layer's first product."""
        for gate, part in ((self.mixer_gate, self.mixer), (self.feed_forward_gate, self.feed_forward)):
            if gate is not None:
                if not hasattr(part, "stack_rows"):
                    raise ValueError(f"{type(part).__name__} cannot carry a gate's rows in its product")
                part.stack_rows(gate.weight)
                gate.weight = None
        self._stacked = True

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool, select_rows: Optional[torch.Tensor]):
        if delta is not None:
            raise RuntimeError("post_norm_residual: the layer before left something to add")
        if not self._stacked:
            self._stack_gates()
        k = ops.kernels()
        x = residual
        history = None
        if self.depth_mix is not None:
            history = ctx.step_cache.setdefault("depth_history", [])
            if not history:
                history.append(x)            # X_0: what the embedding left
        idx = len(history) if history is not None else 0
        if x.dtype == self.dtype:
            x_act = x
        else:
            x_act = ctx.step_cache.get("stream_act")
            if x_act is None or x_act.shape != x.shape:
                # the first layer reads what the embedding left (an exact copy of bfloat16 table rows)
                x_act = ctx.buf("stream_act_in", x.shape, self.dtype)
                k.depth_mix([x], _one(x.device), None, False, None, x_act)
        # ---- mixer, gate, sum, norm ----
        if self.mixer_gate is not None:
            y_sub, g = self.mixer.forward(x_act, ctx, cache, writes_cache, with_extra=True)
            gb = self.mixer_gate.bias
        else:
            y_sub, g, gb = self.mixer.forward(x_act, ctx, cache, writes_cache), None, None
        last = self.feed_forward is None
        name = f"result{idx}" if last else "mid"
        y, y_act = self.mixer_norm.sum_norm(x, self.alpha, y_sub, g, gb, ctx, name, want_act=not last)
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        if not last:
            if gathers:          # the run order's last layer: only the wanted rows go through the feed-forward
                r = select_rows.shape[0]
                y_sel = ctx.buf("mid_rows", (r, y.shape[1]), y.dtype)
                k.gather_rows(y, select_rows, y_sel)
                if y_act is y:
                    y_act_sel = y_sel
                else:
                    y_act_sel = ctx.buf("mid_act_rows", (r, y.shape[1]), y_act.dtype)
                    k.gather_rows(y_act, select_rows, y_act_sel)
                y, y_act = y_sel, y_act_sel
            if self.feed_forward_gate is not None:
                z_sub, g = self.feed_forward.forward(y_act, ctx, with_extra=True)
                gb = self.feed_forward_gate.bias
            else:
                z_sub, g, gb = self.feed_forward.forward(y_act, ctx), None, None
            z, _ = self.feed_forward_norm.sum_norm(y, self.alpha, z_sub, g, gb, ctx, f"result{idx}", want_act=False)
            selected = gathers
        else:
            z = y
            if gathers:
                z_sel = ctx.buf("result_rows", (select_rows.shape[0], z.shape[1]), z.dtype)
                k.gather_rows(z, select_rows, z_sel)
                z = z_sel
            selected = gathers
        if self.depth_mix is None:
            if z.dtype != self.dtype:
                ctx.step_cache.pop("stream_act", None)
            return z, None
        # ---- the stream handed on: a mix of X_0 .. X_idx ----
        terms = history + [z]
        if len(terms) != self.depth_mix.terms:
            raise RuntimeError(f"depth mix of {self.depth_mix.terms} terms after {len(terms) - 1} layers")
        history.append(z)
        out = ctx.buf(f"mixed{idx % 2}", z.shape, torch.float32)
        if self.dtype == torch.float32:
            k.depth_mix(terms, self.depth_mix.coef, select_rows if selected else None, selected, out, None)
            return out, None
        out_act = ctx.buf(f"mixed_act{idx % 2}", z.shape, self.dtype)
        k.depth_mix(terms, self.depth_mix.coef, select_rows if selected else None, selected, out, out_act)
        ctx.step_cache["stream_act"] = out_act
        return out, None


_ONES = {}


def _one(device) -> torch.Tensor:
    t = _ONES.get(device)
    if t is None:
        t = _ONES[device] = torch.ones(1, dtype=torch.float32, device=device)
    return t
