"""Two mixers side by side: both read the same input, and the layer's mixer output is a weighted sum of theirs,

    y = left_scale * left(h) + right_scale * right(h).

Each member is a mixer in its own right (its kind and parameters in ``left`` / ``right``) with a cache of its own: the pair
answers ``cache_need()`` with the tuple of its members' needs and receives a tuple of views (``parts/base.py:
member_cache_id``).  Members that offer ``input_rows()`` have their input products run as ONE product over the stacked rows,
each member then getting its columns.  A member's tensors go under ``left.<name>`` / ``right.<name>``.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .base import MIXERS, Mixer, register_mixer


@register_mixer("side_by_side")
class SideBySide(Mixer):
    """params: ``hidden_size``, ``left`` and ``right`` (PartSpecs of mixers), ``left_scale``, ``right_scale``."""

    NAMES = ("left", "right")

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.scales = (float(p["left_scale"]), float(p["right_scale"]))
        self.members = []
        for name in self.NAMES:
            ms: PartSpec = p[name]
            params = dict(ms.params)
            params.setdefault("buffers", name + "_")          # the members' workspace must not collide
            self.members.append(MIXERS.build(PartSpec(ms.kind, params), dtype, device))
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.members)
        self.w_in = None
        self.cols = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {f"{name}.{local}": ts for name, m in zip(self.NAMES, self.members) for local, ts in m.tensors().items()}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, m in zip(self.NAMES, self.members):
            m.bind({k[len(name) + 1:]: t for k, t in tensors.items() if k.startswith(name + ".")})
        if all(hasattr(m, "input_rows") for m in self.members):
            ws = [m.input_rows() for m in self.members]
            if len({w.dtype for w in ws}) == 1:
                self.w_in = torch.cat(ws, dim=0).contiguous()
                ends = [0]
                for w in ws:
                    ends.append(ends[-1] + w.shape[0])
                self.cols = ends

    def cache_need(self):
        return tuple(m.cache_need() for m in self.members)

    def kernel_libraries(self):
        libs = ("stream_ops", "gemm_simt")
        for m in self.members:
            libs += tuple(m.kernel_libraries())
        return libs

    def graph_plan(self, num_seqs: int, max_ctx: int):
        return tuple(m.graph_plan(num_seqs, max_ctx) for m in self.members)

    def forward(self, x, ctx, cache, writes_cache: bool):
        k = ops.kernels()
        n = x.shape[0]
        views = cache if isinstance(cache, tuple) else (cache,) * len(self.members)
        plans = ctx.graph_plan(self) or (None,) * len(self.members)
        outs = []
        proj = None
        if self.w_in is not None:
            proj = ctx.buf("side_by_side_in", (n, self.w_in.shape[0]), self.dtype)
            k.linear(x, self.w_in, proj)
        for j, m in enumerate(self.members):
            kw = {}
            if proj is not None:
                kw["proj"] = proj[:, self.cols[j]: self.cols[j + 1]]
            if plans[j] is not None:
                kw["plan"] = plans[j]
            outs.append(m.forward(x, ctx, views[j], writes_cache, **kw))
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.weighted_sum2(outs[0], self.scales[0], outs[1], self.scales[1], out)
        return out
