"""Token embedding and output head.

Embedding: ``x0[t] = E[token_t]`` (src/iian/graph.cpp:39-46); the residual stream it starts is
float32.  Head: ``logits = Wout x`` in float32 on the rows asked for (src/iian/graph.cpp:360-376);
with tied embeddings ``Wout`` is the embedding table itself (src/iian/arch/qwen3.cpp:26-27).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Embedding, Head, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``; optional ``scale`` (default 1): the table row is multiplied by it, in
    float32; optional ``side_width`` (default 0): a second table [vocab, side_width] indexed by the same token ids, whose
    rows the layers read slice by slice (``parts/block.py: TokenSide``); the part only holds it and hands it on through
    ``ctx.step_cache["token_side_table"]``."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.side_width = int(spec.params.get("side_width", 0))
        self.weight: Optional[torch.Tensor] = None
        self.side: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"weight": TensorSpec((self.vocab, self.hidden))}
        if self.side_width:
            t["side"] = TensorSpec((self.vocab, self.side_width))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()
        if self.side_width:
            self.side = tensors["side"].contiguous()

    def kernel_libraries(self):
        return ("elementwise",) + (("stream_ops",) if self.scale != 1.0 else ())

    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buf("residual", (tokens.shape[0], self.hidden), torch.float32)
        if self.side is not None:
            ctx.step_cache["token_side_table"] = self.side
        if self.scale != 1.0:
            ops.kernels().embedding_scaled(self.weight, tokens, self.scale, out)
        else:
            ops.kernels().embedding(self.weight, tokens, out)
        return out


@register_head("lm_head")
class LMHead(Head):
    """params: ``hidden_size``, ``vocab_size``, ``tied`` (use the embedding table); optional ``softcap`` (None or c > 0:
    the logits become ``c tanh(logits / c)``)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        cap = spec.params.get("softcap")
        self.softcap = float(cap) if cap else None
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError("lm_head: softcap must be positive")
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {} if self.tied else {"weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def kernel_libraries(self):
        return ("gemm_simt",) + (("residual_ops",) if self.softcap is not None else ())

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = ctx.buf("logits", (x.shape[0], self.vocab), torch.float32)
        ops.kernels().linear(x, self.weight, logits)
        if self.softcap is not None:
            ops.kernels().tanh_cap(logits, self.softcap)
        return logits
