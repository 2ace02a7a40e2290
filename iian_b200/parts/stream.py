"""Parts that work on the whole residual stream between two layers (``LayerCall.before``).

``add_embedding``: ``x <- x + e`` with ``e`` what the embedding left.  Nothing is launched for it where the block before left
a ``NormedAddend``: ``e`` rides as the second addend of the sum the next norm does anyway.

``reinject_embedding``: ``x <- W [x ; e]`` with ``e`` what the embedding left and ``W`` [hidden, 2 hidden] (the columns
that meet ``x`` first).  A model that runs a stretch of its layers several times puts it before the first layer of every
run, so that each run sees the input again.  The sum that is still owed to the stream (``delta``) is added while the
product's input is put together; the product writes the new float32 stream into a buffer of its own, so what the
embedding left stays as it was.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import NormedAddend, StreamPart, register_stream_part


@register_stream_part("reinject_embedding")
class EmbeddingReinjection(StreamPart):
    """params: ``hidden_size``."""

    needs_embedding_out = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.weight = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden, 2 * self.hidden))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self):
        return ("stream_ops", "gemm_simt")

    def forward(self, residual: torch.Tensor, delta, ctx):
        k = ops.kernels()
        e = ctx.step_cache["embedding_out"]
        d1, d2 = delta if isinstance(delta, tuple) else (delta, None)
        n = residual.shape[0]
        both = ctx.buf("reinject_in", (n, 2 * self.hidden), self.dtype)
        k.stream_concat(residual, d1, d2, e, both)
        # the stream moves to another buffer than the one it came in (and never into the one the embedding wrote)
        turn = ctx.step_cache.get("reinject_turn", 0)
        ctx.step_cache["reinject_turn"] = turn + 1
        out = ctx.buf(f"reinjected{turn % 2}", (n, self.hidden), torch.float32)
        k.linear(both, self.weight, out)
        return out, None


@register_stream_part("add_embedding")
class EmbeddingAddition(StreamPart):
    """``x <- x + e``, in float32.  No tensors, no parameters."""

    needs_embedding_out = True

    def kernel_libraries(self):
        return ("residual_ops",)

    def forward(self, residual: torch.Tensor, delta, ctx):
        e = ctx.step_cache["embedding_out"]
        if delta is None:
            return residual, NormedAddend(None, None, 0.0, extra=e)
        if isinstance(delta, NormedAddend) and delta.extra is None:
            return residual, NormedAddend(delta.y, delta.weight, delta.eps, extra=e)
        raise ValueError("add_embedding: the block before must leave nothing or one normalised addend to the stream")
