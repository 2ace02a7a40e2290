"""Shared by the Nogelorn tests: small configurations that differ in every size and option, model folders with random
weights in temporary places, and the comparison of replayed logits with the plain implementation
(tests/plain_nogelorn.py)."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

import plain_nogelorn as plain

F64 = torch.float64


def rot(dims, base, **scaling):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def window_attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rotation=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotation:
        m["rot"] = rotation
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def attention(*a, **kw):
    return {"type": "attention", "mixer": window_attention(*a, **kw)}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def parallel(left, right_heads, right_dim, right_vdim, tau, rank, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                          "right": {"heads": right_heads, "dim": right_dim, "vdim": right_vdim, "tau": tau,
                                                    "decay_rank": rank}}}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# G: odd sizes everywhere; the repeated stretch starts behind the first layer and is followed by another; values wider and
#    narrower than keys; partial rotation with all three wavelength bands; a ramp that ends early; kept keys that are no
#    multiple of the page; 3:1 and 1:1 grouping; a layer without feed-forward; one, two and three experts per token; an
#    expert every token uses, and none.
# H: sizes the bfloat16 fast products take (multiples of 32); the first layer alone runs three times; attention heads of 64
#    (the tensor-core attention in bfloat16) with a sink and a gate but NO kept keys; a window of 33; a recurrence wider than
#    it is deep.
# I: no repetition; one head everywhere; a window shorter than a page with more kept keys than the window is long, and one
#    longer than any request; no rotation in one layer and a plain one (no rescaling) in another; a recurrence deep enough
#    for 32 lanes per column; every expert chosen; no embedding factor.
# J: heads of 128: kept keys (the general kernel), a left member of 128 (tcgen05 for portions), a recurrence 128 deep; the
#    first two layers run twice.    Q: a width and sizes that are multiples of 4 only.
CONFIGS = {
    "G": {"architecture": "Nogelorn", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
          "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        layer(lightning(3, 24, 40, [0.9, 0.5, 0.99]), moe(5, 2, 48, shared=40)),
        layer(parallel(window_attention(6, 2, 16, 24, 0.3, window=24,
                                        rotation=rot(8, 30000.0, factor=8.0, low=1.0, high=4.0, original=256)),
                       3, 24, 16, 8.0, 12, 0.7, 1.1), None),
        layer(attention(4, 4, 24, 16, 0.2, window=17, keep_first=5,
                        rotation=rot(24, 10000.0, factor=4.0, original=32, fast=16.0, slow=2.0)), moe(6, 1, 32)),
        layer(lightning(2, 16, 24, [0.7, 0.97]), moe(4, 3, 24, shared=56))]},
    "H": {"architecture": "Nogelorn", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.0},
          "loop": {"start": 0, "stop": 1, "times": 3}, "layers": [
        layer(attention(8, 2, 64, 64, 0.11, window=33, keep_first=0,
                        rotation=rot(32, 500000.0, factor=2.0, original=64, fast=8.0, slow=1.0)), moe(8, 2, 64, shared=96)),
        layer(parallel(window_attention(8, 2, 64, 64, 0.125, window=40,
                                        rotation=rot(64, 10000.0, factor=4.0, low=1.0, high=2.0, original=128)),
                       2, 32, 64, 16.0, 8, 0.5, 0.8), moe(8, 1, 64)),
        layer(lightning(2, 64, 128, [0.61, 0.999]), moe(8, 3, 64, shared=32))]},
    "I": {"architecture": "Nogelorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        layer(attention(1, 1, 8, 12, 0.4, window=5, keep_first=9, rotation=rot(8, 100.0)), moe(2, 2, 32, shared=16)),
        layer(lightning(1, 160, 16, [0.95]), None),
        layer(parallel(window_attention(2, 1, 32, 32, 0.2, window=500), 1, 8, 8, 2.0, 4, 1.0, 1.0), moe(3, 1, 16)),
        layer(attention(2, 2, 16, 8, 0.25), None)]},
}
CONFIGS["J"] = {"architecture": "Nogelorn", "vocab": 331, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
                "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    layer(attention(4, 2, 128, 128, 0.09, window=40, keep_first=16,
                    rotation=rot(128, 1000000.0, factor=4.0, original=64, fast=32.0, slow=1.0)), moe(4, 2, 64, shared=64)),
    layer(parallel(window_attention(4, 1, 128, 128, 0.088, window=90, rotation=rot(64, 500000.0)),
                   2, 128, 64, 4.0, 16, 0.6, 0.9), moe(6, 1, 128)),
    layer(lightning(2, 128, 64, [0.8, 0.995]), moe(4, 2, 32, shared=128))]}
CONFIGS["Q"] = {"architecture": "Nogelorn", "vocab": 150, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 7.0},
                "loop": {"start": 1, "stop": 2, "times": 3}, "layers": [
    layer(lightning(5, 20, 12, [0.5, 0.6, 0.7, 0.8, 0.9]), moe(3, 2, 36, shared=20)),
    layer(attention(5, 1, 20, 12, 0.25, window=9, keep_first=2, rotation=rot(10, 1000.0, factor=3.0, original=16, fast=4.0, slow=1.0)),
          moe(3, 2, 36)),
    layer(parallel(window_attention(3, 3, 12, 20, 0.3, window=11, rotation=rot(12, 5000.0, factor=2.0, low=1.0, high=8.0, original=40)),
                   5, 12, 20, 5.0, 4, 0.4, 1.3), None)]}
BLOCK_SIZE = {"G": 16, "H": 8, "I": 32, "J": 16, "Q": 16}
SEED = {"G": 31, "H": 32, "I": 33, "J": 34, "Q": 35}


def write_case(tmp_path, name: str, store_dtype=torch.bfloat16, std: float = 0.08, config=None, router_step: float = 0.0) -> str:
    """A model folder of configuration ``name`` with random weights.  ``std`` is large enough that attention weights, gates
    and decays are far from uniform.  ``router_step`` > 0: the routers' biases are set that far apart
    (``spread_router_biases``)."""
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder
    arch = get_architecture("Nogelorn")
    d = os.path.join(str(tmp_path), f"nogelorn{name}_{str(store_dtype).split('.')[-1]}" + ("_steady" if router_step else ""))
    if not os.path.isdir(d):
        write_model_folder(d, arch, arch.load_config(config or CONFIGS[name]), seed=SEED.get(name, 1), store_dtype=store_dtype,
                           std=std, norm_jitter=0.3)
        if router_step:
            spread_router_biases(d, store_dtype, router_step)
    return d


def spread_router_biases(model_dir: str, store_dtype, step: float) -> None:
    """Random router weights put the logits of a few experts within a hair of each other for a good part of the tokens, and
    16-bit rounding of the router's input then decides which expert a token takes -- with a norm behind the feed-forward, a
    different expert is a different output at full size, for that token and, through the mixers, for those right behind it.
    So for the bfloat16 runs of whole models the routers' biases are set ``step`` apart (in a shuffled order that differs from
    layer to layer): ties are rare.  The 32-bit runs and the kernels' own tests keep routers that the input moves freely."""
    from iian_b200.weights.safetensors_io import write_safetensors
    w = plain.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    for i, name in enumerate(sorted(k for k in w if k.endswith(".router.b"))):
        n = w[name].numel()
        order = torch.randperm(n, generator=torch.Generator().manual_seed(100 + i)).to(torch.float32)
        w[name] = (order - (n - 1) / 2) * step
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      {k: (v.to(store_dtype) if v.is_floating_point() else v) for k, v in w.items()}, metadata={"format": "pt"})


def plain_logits(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_folder(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}


def rounded_plain(folder, reqs, dtype: torch.dtype):
    """The plain implementation with the input and the result of every matrix product rounded to ``dtype``: how far rounding
    alone moves the logits at each position."""
    cfg, w = plain.load_folder(folder)
    plain.product_rounding = lambda z: z.to(dtype).to(F64)
    try:
        return {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    finally:
        plain.product_rounding = None


def router_margins(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    """Per request and position the smallest gap, over all layer runs, between the last expert a router takes and the best
    one it leaves out.  Where the gap is within a reduced precision's rounding of the logits the choice may fall the other
    way, and with it the whole (normalised) feed-forward output of that token: such positions say nothing about a kernel."""
    cfg, w = plain.load_folder(model_dir)
    out = {}
    for rid, toks in requests.items():
        plain.router_margins = []
        try:
            plain.forward(cfg, w, toks)
            out[rid] = torch.stack(plain.router_margins).min(0).values if plain.router_margins else torch.full((len(toks),), float("inf"))
        finally:
            plain.router_margins = None
    return out
