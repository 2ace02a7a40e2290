"""Shared by the Senadra tests: small configurations that differ in every size and option, model folders with random
weights in temporary places, and the comparison of replayed logits with the plain implementation
(tests/plain_senadra.py)."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

import plain_senadra as plain


def attention(heads, kv_heads, dim, vdim, chunk, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                   "q_rank": q_rank, "scale": scale, "rot": {"dims": rot_dim, "base": base}}}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# P: odd sizes everywhere; three query heads on one key/value head, values wider than keys; a layer that reads the first
#    layer's keys and values under a chunk size of its own; two query/key heads for four value heads in the recurrence, four
#    taps, low-rank maps of different sizes (none equal to the side input's); a layer without feed-forward; chunks that are no
#    multiple of the page.
# Q: sizes the bfloat16 fast products take (multiples of 32); attention heads of 64 with values of 64; a reader of the
#    SECOND layer's cache; one query/key head for four value heads; latent values narrower than its keys.
# R: one head everywhere; a convolution of one tap (no tail); a chunk shorter than a page and one longer than any request; no
#    side input, no cap on the logits, no factor on the residual; a recurrence deep enough for the many-entries-per-lane form.
# S: heads of 128 with values of 128; a latent of 128; a recurrence 128 deep and wide; two readers of one cache.
# T: a width and sizes that are multiples of 4 only (no 16-byte rows for the fast products); values narrower than keys.
CONFIGS = {
    "P": {"architecture": "Senadra", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.45,
          "token_side": {"dim": 10}, "logit_softcap": 8.0, "layers": [
        layer(attention(6, 2, 16, 24, 24, 0.3), dense(160)),
        layer(delta(4, 2, 12, 20, 4, 6, 9), dense(64)),
        layer(latent(3, 16, 8, 24, 40, 28, 0.2, 30000.0), None),
        layer(attention(6, 2, 16, 24, 17, 0.25, kv_from=0), dense(48)),
        layer(delta(2, 2, 40, 8, 2, 5, 3), None)]},
    "Q": {"architecture": "Senadra", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
          "token_side": {"dim": 32}, "logit_softcap": 30.0, "layers": [
        layer(latent(4, 32, 32, 16, 64, 64, 0.125), dense(256)),
        layer(attention(4, 4, 64, 64, 33, 0.11), dense(128)),
        layer(attention(8, 4, 64, 64, 50, 0.12, kv_from=1), None),
        layer(delta(4, 1, 64, 32, 3, 32, 32), dense(256)),
        layer(attention(8, 2, 32, 64, 70, 0.2), dense(64))]},
    "R": {"architecture": "Senadra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "layers": [
        layer(delta(1, 1, 160, 16, 1, 7, 2), dense(32)),
        layer(attention(1, 1, 8, 8, 5, 0.4), None),
        layer(latent(1, 8, 4, 8, 16, 12, 0.3), dense(64)),
        layer(attention(2, 1, 32, 16, 500, 0.2), dense(32)),
        layer(attention(2, 2, 16, 32, None, 0.3), None)]},
}
CONFIGS["S"] = {"architecture": "Senadra", "vocab": 331, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 0.25,
                "token_side": {"dim": 16}, "logit_softcap": 20.0, "layers": [
    layer(attention(4, 2, 128, 128, 40, 0.09), dense(384)),
    layer(delta(2, 2, 128, 128, 3, 16, 24), dense(256)),
    layer(attention(4, 2, 128, 128, 90, 0.07, kv_from=0), dense(128)),
    layer(latent(4, 64, 64, 64, 128, 96, 0.09, 500000.0), None),
    layer(attention(2, 2, 128, 128, 64, 0.1, kv_from=0), dense(128))]}
CONFIGS["T"] = {"architecture": "Senadra", "vocab": 150, "width": 100, "norm": {"eps": 1e-5}, "residual_mult": 1.5,
                "token_side": {"dim": 4}, "logit_softcap": 5.0, "layers": [
    layer(delta(5, 5, 20, 12, 3, 4, 4), dense(52)),
    layer(attention(5, 1, 20, 12, 9, 0.25), dense(36)),
    layer(latent(5, 12, 4, 20, 36, 20, 0.3), None)]}
BLOCK_SIZE = {"P": 16, "Q": 8, "R": 32, "S": 16, "T": 16}
SEED = {"P": 31, "Q": 32, "R": 33, "S": 34, "T": 35}


def write_case(tmp_path, name: str, store_dtype=torch.bfloat16, std: float = 0.08) -> str:
    """A model folder of configuration ``name`` with random weights.  ``std`` is large enough that attention weights and
    gates are far from uniform."""
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder
    arch = get_architecture("Senadra")
    d = os.path.join(str(tmp_path), f"senadra{name}_{str(store_dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_model_folder(d, arch, arch.load_config(CONFIGS[name]), seed=SEED[name], store_dtype=store_dtype, std=std,
                           norm_jitter=0.3)
    return d


def plain_logits(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_folder(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}
