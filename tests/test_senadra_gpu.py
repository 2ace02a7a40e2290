"""Senadra on the GPU.  Each new kernel alone against the plain functions of tests/plain_senadra.py (the scaled residual sum
with the norm, the normalised addend, the gated token-indexed factor, xIELU, the tanh cap; keys and normalised values into
pages whose value cells have a size of their own; attention inside chunks with a stand-out key just inside and just outside
a chunk's edge, at page borders and far back, in portions and as single tokens; the delta-rule scan at every depth, cut into
steps, with slots used again; the latent mixer with a query latent, interleaved rotation and an output gate); then whole
models under every way of cutting the work, in 32-bit and in bfloat16, layer by layer and at the logits; greedy generation
through the engine's entry point with and without CUDA graphs; the trace runner as a program."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_senadra as plain
from helpers import max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from senadra_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def K():
    from iian_b200 import ops
    return ops.kernels()


def close(got, want, dtype, what, rel16=2e-2, abs32=2e-5):
    got, want = got.double().cpu(), want.double().cpu()
    tol = abs32 * max(1.0, want.abs().max().item()) if dtype == "float32" else rel16 * want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= tol, f"{what} [{dtype}]: max error {err:.3g} > {tol:.3g}"


# ---- row-wise kernels ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scaled_sums_norms_and_activations(dtype):
    g = torch.Generator().manual_seed(1)
    for h in (72, 1000, 4100):
        x = torch.randn(5, h, generator=g) * 3
        d = torch.randn(5, h, generator=g).to(DT[dtype])
        w = torch.randn(h, generator=g)
        res = x.to(DEV).clone()
        normed = torch.empty(5, h, device=DEV, dtype=DT[dtype])
        copy = torch.empty(5, h, device=DEV, dtype=DT[dtype])
        K().scaled_add_rms_norm(res, d.to(DEV), 0.37, w.to(DEV), 1e-5, normed, copy)
        s = x.double() + 0.37 * d.double()
        close(res, s, "float32", f"stream after the scaled sum, width {h}")
        close(normed, plain.rms_norm(s, w.double(), 1e-5), dtype, f"norm of the new stream, width {h}", rel16=8e-3)
        close(copy, s, dtype, "the stream's copy", rel16=5e-3)
        res = x.to(DEV).clone()
        K().scaled_add_rms_norm(res, None, 0.37, w.to(DEV), 1e-5, normed)              # the first norm of a model: nothing to add
        close(res, x, "float32", "stream without an addend", abs32=0.0)
        close(normed, plain.rms_norm(x.double(), w.double(), 1e-5), dtype, "norm alone", rel16=8e-3)
        y = (torch.randn(5, h, generator=g) * 7).to(DT[dtype])
        res = x.to(DEV).clone()
        K().scaled_add_unit_rms(res, y.to(DEV), 1.7, w.to(DEV), 1e-5)
        close(res, x.double() + 1.7 * plain.rms_norm(y.double(), w.double(), 1e-5), "float32", f"normalised addend, width {h}")
    wide = (torch.randn(6, 100, generator=g) * 2).to(DT[dtype])
    w = torch.randn(60, generator=g)
    out = torch.empty(6, 60, device=DEV, dtype=DT[dtype])
    K().rms_norm_rows(wide.to(DEV)[:, 30:90], w.to(DEV), 1e-6, out)
    close(out, plain.rms_norm(wide.double()[:, 30:90], w.double(), 1e-6), dtype, "norm of a column slice", rel16=8e-3)
    z = (torch.randn(7, 333, generator=g) * 3).to(DT[dtype])
    pq = torch.tensor([0.4, -1.3])
    out = torch.empty(7, 333, device=DEV, dtype=DT[dtype])
    K().xielu(z.to(DEV), pq.to(DEV), out)
    close(out, plain.xielu(z.double(), pq[0].double(), pq[1].double()), dtype, "xIELU", rel16=8e-3)
    lg = torch.randn(3, 500, generator=g) * 40
    dev = lg.to(DEV).clone()
    K().tanh_cap(dev, 11.0)
    close(dev, plain.tanh_cap(lg.double(), 11.0), "float32", "tanh cap")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_indexed_factor(dtype):
    g = torch.Generator().manual_seed(2)
    vocab, dim, layers, n = 40, 10, 3, 9
    table = torch.randn(vocab, dim * layers, generator=g).to(DT[dtype])
    tokens = torch.randint(0, vocab, (n,), generator=g).to(torch.int32)
    gate = (torch.randn(n, dim, generator=g) * 2).to(DT[dtype])
    out = torch.empty(n, dim, device=DEV, dtype=DT[dtype])
    for layer in range(layers):
        K().gelu_mul_table(gate.to(DEV), table.to(DEV), layer * dim, tokens.to(DEV), None, out)
        want = plain.gelu_tanh(gate.double()) * table.double()[tokens.long()][:, layer * dim:(layer + 1) * dim]
        close(out, want, dtype, f"gelu times the token's entries of layer {layer}", rel16=1e-2)
    rows = torch.tensor([8, 0, 4], dtype=torch.int32)                                  # selected rows: row r belongs to token rows[r]
    out3 = torch.empty(3, dim, device=DEV, dtype=DT[dtype])
    K().gelu_mul_table(gate[:3].contiguous().to(DEV), table.to(DEV), dim, tokens.to(DEV), rows.to(DEV), out3)
    want = plain.gelu_tanh(gate[:3].double()) * table.double()[tokens.long()[rows.long()]][:, dim:2 * dim]
    close(out3, want, dtype, "selected rows", rel16=1e-2)


# ---- attention inside chunks ---------------------------------------------------------------------------
def _fill_pages(dtype, nh, nkv, dk, dv, n, page, seed, eps=1e-5):
    """Projections q | gate | k | v of n tokens of one sequence, keys and normalised values through the store kernel into
    scattered pages; returns what the plain functions make of the same rows."""
    g = torch.Generator().manual_seed(seed)
    front = nh * dk + nh * dv
    width = front + nkv * dk + nkv * dv
    proj = torch.randn(n, width, generator=g).to(DT[dtype])
    n_used = -(-n // page)
    order = torch.randperm(n_used + 3, generator=g)[:n_used].to(torch.int32)
    kc = torch.zeros(n_used + 3, nkv, page, dk, dtype=DT[dtype], device=DEV)
    vc = torch.zeros(n_used + 3, nkv, page, dv, dtype=DT[dtype], device=DEV)
    pos = torch.arange(n, dtype=torch.int32)
    slots = (order[(pos // page).long()] * page + pos % page).to(torch.int32)
    K().kv_store_normed(proj.to(DEV), front, front + nkv * dk, kc, vc, slots.to(DEV), num_kv_heads=nkv, k_dim=dk, v_dim=dv, eps=eps,
                        norm_values=True)
    p64 = proj.double()
    k = p64[:, front:front + nkv * dk].view(n, nkv, dk)
    v = plain.unit_rms(p64[:, front + nkv * dk:].view(n, nkv, dv), eps)
    return SimpleNamespace(proj=proj, kc=kc, vc=vc, order=order, slots=slots, pos=pos, q=p64[:, :nh * dk].view(n, nh, dk).clone(),
                           gate=p64[:, nh * dk:front], k=k.clone(), v=v, front=front)


def _plain_chunked(c, nh, nkv, scale, chunk, r1, r2):
    n = c.q.shape[0]
    group = torch.arange(nh) // (nh // nkv)
    scores = torch.einsum("ihd,jhd->hij", c.q, c.k[:, group]) * scale - plain.distance_penalty(n, r1, r2)
    p = plain.masked_softmax(scores, plain.chunk_mask(n, chunk)[None])
    o = torch.einsum("hij,jhd->ihd", p, c.v[:, group]).reshape(n, -1)
    return o * torch.sigmoid(c.gate), p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, dk, dv", [(6, 2, 16, 24), (4, 4, 64, 64), (8, 2, 64, 32), (2, 1, 128, 128), (3, 1, 24, 40),
                                              (4, 2, 128, 96), (5, 5, 20, 12)])
def test_values_are_cached_divided_by_their_root_mean_square(dtype, nh, nkv, dk, dv):
    page = 8
    c = _fill_pages(dtype, nh, nkv, dk, dv, 21, page, seed=dk + dv)
    cells = c.slots.long().to(DEV)
    k_got = c.kc.permute(0, 2, 1, 3).reshape(-1, nkv, dk)[cells]
    v_got = c.vc.permute(0, 2, 1, 3).reshape(-1, nkv, dv)[cells]
    assert torch.equal(k_got.cpu().double(), c.k), "keys are cached as projected"
    close(v_got, c.v, dtype, "values in their cells", rel16=8e-3)
    assert int((c.kc != 0).any(-1).any(1).sum()) == 21, "cells of other tokens were written"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, dk, dv, chunk, page", [(6, 2, 16, 24, 37, 16), (4, 4, 64, 64, 33, 8), (8, 2, 64, 32, 64, 16),
                                                          (2, 1, 128, 128, None, 32), (3, 1, 24, 40, 5, 16), (4, 2, 128, 128, 150, 16),
                                                          (4, 2, 128, 96, 700, 32), (2, 2, 64, 64, 1, 16)])
def test_attention_sees_its_chunk_exactly(dtype, nh, nkv, dk, dv, chunk, page):
    """Two keys are made to stand out for the last tokens' queries: the FIRST position of the last token's chunk (the
    farthest key it sees) and the position just before it (the nearest it must not see; the last token of the chunk before
    does).  Without a chunk: position 1, far back.  Queries: a portion of the last tokens, single tokens, the first ones, a
    long portion over several chunk edges."""
    n = 300 if chunk and chunk < 300 else 1500
    c = _fill_pages(dtype, nh, nkv, dk, dv, n, page, seed=nh * dk + dv)
    first = ((n - 1) // chunk) * chunk if chunk else 1
    before = first - 1 if chunk and first > 0 else -1
    first_of_group = torch.arange(nkv) * (nh // nkv)
    for j, asker in ((first, n - 1), (before, before)):
        if j < 0 or (chunk == 1):
            continue
        key = (2.5 * c.q[asker, first_of_group]).to(DT[dtype])
        cell = int(c.slots[j])
        c.kc[cell // page, :, cell % page, :] = key.to(DEV)
        c.k[j] = key.double()
    r1 = torch.rand(nh, generator=torch.Generator().manual_seed(5)) * 0.4
    r2 = torch.rand(nh, generator=torch.Generator().manual_seed(6)) * 2 + 0.1
    scale = 2.0 / math.sqrt(dk)
    want, p = _plain_chunked(c, nh, nkv, scale, chunk, r1.double(), r2.double())
    if chunk != 1:
        assert p[:, n - 1, first].max() > 0.2, "the stand-out key at the chunk's start must matter"
    if before >= 0 and chunk != 1:
        assert p[:, n - 1, before].max() == 0 and p[:, before, before].max() > 0.2
    no_penalty, _ = _plain_chunked(c, nh, nkv, scale, chunk, torch.zeros(nh, dtype=F64), r2.double())
    if chunk != 1:
        assert (no_penalty - want).abs().max() > 1e-3, "the penalty must show"
    bt = torch.full((1, max(64, c.order.numel())), -1, dtype=torch.int32)
    bt[0, : c.order.numel()] = c.order
    dev_proj = c.proj.to(DEV)
    lo = max(0, n - 200)
    for rows in (list(range(n - 7, n)), [n - 2], [n - 1], [max(before, 0)], list(range(0, 3)), list(range(lo, n)), list(range(0, 130))):
        r = torch.tensor(rows)
        meta = SimpleNamespace(positions=c.pos[r].to(DEV), seq_of_token=torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                               cu_q=torch.tensor([0, len(rows)], dtype=torch.int32, device=DEV),
                               ctx_len=torch.tensor([rows[-1] + 1], dtype=torch.int32, device=DEV), block_table=bt.to(DEV),
                               slots=c.slots[r].to(DEV), num_seqs=1, num_tokens=len(rows), max_q_len=len(rows), max_ctx=rows[-1] + 1,
                               decode_only=len(rows) == 1, h_q_len=[len(rows)], h_ctx_len=[rows[-1] + 1])
        sel = dev_proj[r.to(DEV)]
        out = torch.empty(len(rows), nh * dv, dtype=DT[dtype], device=DEV)
        K().chunked_attention(sel[:, : nh * dk], c.kc, c.vc, out, meta, num_heads=nh, num_kv_heads=nkv, k_dim=dk, v_dim=dv, scale=scale,
                              chunk=chunk, window=None, r1=r1.to(DEV), r2=r2.to(DEV), gate=sel[:, nh * dk: c.front])
        close(out, want[r], dtype, f"attention rows {rows[0]}..{rows[-1]}", rel16=2.5e-2)
        if len(rows) == 1 and K().chunked_attention_mma_ok(DT[dtype], nh, nkv, dk, dv, scale):
            # the decode form with its keys unsplit, merged inside a cluster and merged through scratch memory
            for parts in (1, 2, 3, 4):
                out.zero_()
                K().chunked_attention(sel[:, : nh * dk], c.kc, c.vc, out, meta, num_heads=nh, num_kv_heads=nkv, k_dim=dk, v_dim=dv,
                                      scale=scale, chunk=chunk, window=None, r1=r1.to(DEV), r2=r2.to(DEV),
                                      gate=sel[:, nh * dk: c.front], n_split=parts)
                close(out, want[r], dtype, f"attention row {rows[0]} in {parts} key parts", rel16=2.5e-2)


# ---- the delta-rule scan ------------------------------------------------------------------------------------------
def _selectors(H, G, D, V, taps, g):
    """Tensors that make the plain mixer read its projections straight out of the columns of its input
    [q | k | v | b | z | gate]: every weight matrix picks columns, the output projection is the identity."""
    GD, HV, HD = G * D, H * V, H * D
    width = 2 * GD + HV + H + HD + HV
    eye = torch.eye(width, dtype=F64)
    off = [0, GD, 2 * GD, 2 * GD + HV, 2 * GD + HV + H, 2 * GD + HV + H + HD, width]
    t = {"q": eye[off[0]:off[1]], "k": eye[off[1]:off[2]], "v": eye[off[2]:off[3]], "b": eye[off[3]:off[4]],
         "a1": eye[off[4]:off[5]], "a2": torch.eye(HD, dtype=F64), "g1": eye[off[5]:off[6]], "g2": torch.eye(HV, dtype=F64),
         "o": torch.eye(HV, dtype=F64)}
    r = lambda *s: torch.randn(*s, generator=g)
    t["q.conv"], t["k.conv"], t["v.conv"] = r(GD, taps), r(GD, taps), r(HV, taps)
    t["A_log"], t["dt_bias"], t["norm"] = r(H) * 0.5, r(HD), r(V)
    return t, off


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, V, taps", [(4, 2, 12, 20, 4), (2, 2, 40, 8, 2), (4, 1, 64, 32, 3), (1, 1, 160, 16, 1), (2, 2, 128, 128, 3),
                                              (5, 5, 20, 12, 3), (1, 1, 8, 8, 8), (1, 1, 300, 6, 2), (6, 3, 32, 64, 4)])
def test_delta_rule_cut_into_steps_with_slots_used_again(dtype, H, G, D, V, taps):
    plan = [[(0, 0, 5), (1, 0, 1)], [(0, 5, 7)], [(0, 7, 8)], [(0, 8, 37)], [(2, 0, 2)], [(2, 2, 3)], [(2, 3, 12)]]
    _delta_plan(dtype, H, G, D, V, taps, [37, 1, 12], plan)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, V, taps", [(4, 2, 12, 20, 4), (2, 2, 128, 128, 3), (1, 1, 300, 6, 2), (6, 3, 32, 64, 4), (2, 1, 64, 32, 1)])
@pytest.mark.parametrize("big", [(300, 270), (700, 590)])
def test_delta_rule_steps_of_many_tokens(dtype, H, G, D, V, taps, big):
    """Steps long enough for the preparation's tiled form (rows staged through shared memory), with a sequence that starts in
    the middle of a tile, behind and ahead of short steps; in 32-bit the long steps give the bits the short ones give."""
    a, b = big
    plan = [[(0, 0, 3), (1, 0, 5)], [(0, 3, a), (2, 0, b)], [(2, b, b + 20)], [(0, a, a + 1), (2, b + 20, b + 21)]]
    got = _delta_plan(dtype, H, G, D, V, taps, [a + 1, 5, b + 21], plan, slots=(2, 0, 1))
    if dtype == "float32":
        short = [[(0, 0, 3), (1, 0, 5)]] + [[(0, lo, min(lo + 100, a))] for lo in range(3, a, 100)] + \
                [[(2, lo, min(lo + 90, b + 20))] for lo in range(0, b + 20, 90)] + [[(0, a, a + 1), (2, b + 20, b + 21)]]
        again = _delta_plan(dtype, H, G, D, V, taps, [a + 1, 5, b + 21], short, compare=False, slots=(2, 0, 1))
        for s in range(3):
            assert torch.equal(got[s], again[s]), f"sequence {s}: long and short steps differ by {(got[s] - again[s]).abs().max()}"


def _delta_plan(dtype, H, G, D, V, taps, lens, plan, compare=True, slots=(2, 0, 2)):
    g = torch.Generator().manual_seed(H * D + V + taps)
    t, off = _selectors(H, G, D, V, taps, g)
    mc = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "conv": taps}
    eps = 1e-5
    n_state = K().delta_state_floats(H, G, D, V, taps)
    state = torch.full((3, n_state), 7.0, device=DEV)                                 # slots hold leftovers ...
    seqs, wants = [], []
    for L in lens:
        proj = (torch.randn(L, off[4], generator=g) * 1.5).to(DT[dtype])              # q | k | v | b
        z = torch.randn(L, H * D, generator=g) * 2
        gate = (torch.randn(L, H * V, generator=g) * 2).to(DT[dtype])
        seqs.append((proj, z, gate))
        h = torch.cat([proj.double(), z.double(), gate.double()], dim=1)
        wants.append(plain.channel_delta(h, t, "", mc, eps, return_state=True) if compare else None)
    conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]]).to(DEV)
    norm_w = t["norm"].repeat(H).to(DEV)
    # by default the third sequence inherits the first one's slot
    got = [[] for _ in lens]
    fresh = {0: True, 1: True, 2: True}
    bufs = {}

    def buf(name, shape, dt):
        key = (name, tuple(shape), dt)
        if key not in bufs:
            bufs[key] = torch.empty(shape, dtype=dt, device=DEV)
        return bufs[key]
    for step in plan:
        rows, cu, sl, seq_of = [[], [], []], [0], [], []
        for j, (s, lo, hi) in enumerate(step):
            if fresh[s]:
                state[slots[s]].zero_()                                                # ... and are zeroed when a request takes them
                fresh[s] = False
            for a, src in zip(rows, seqs[s]):
                a.append(src[lo:hi])
            cu.append(cu[-1] + hi - lo)
            sl.append(slots[s])
            seq_of += [j] * (hi - lo)
        # a padding sequence (slot -1) rides along: it must change nothing and yield zeros
        for a, src in zip(rows, seqs[0]):
            a.append(src[:1])
        cu.append(cu[-1] + 1); sl.append(-1); seq_of.append(-1)
        proj, z, gate = (torch.cat(a).to(DEV) for a in rows)
        ctx = SimpleNamespace(cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), buf=buf,
                              seq_of_token=torch.tensor(seq_of, dtype=torch.int32, device=DEV),
                              state_slots=torch.tensor(sl, dtype=torch.int32, device=DEV))
        heads = torch.full((proj.shape[0], H * V), 9.0, device=DEV)
        K().delta_rule(proj, 0, off[3], z, conv_w, t["A_log"].to(DEV), t["dt_bias"].to(DEV), state, ctx, heads, num_heads=H,
                       num_kv_heads=G, dim=D, v_dim=V)
        assert heads[cu[-2]:].abs().max() == 0
        normed = torch.empty(proj.shape[0], H * V, device=DEV, dtype=DT[dtype])
        K().head_norm_gate(heads, norm_w, gate, normed, num_heads=H, eps=eps)
        for j, (s, lo, hi) in enumerate(step):
            got[s].append(normed[cu[j]:cu[j + 1]].cpu())
    got = [torch.cat(x) for x in got]
    if not compare:
        return got
    for s in range(3):
        close(got[s], wants[s][0], dtype, f"sequence {s} of {H} heads {D} x {V}", rel16=1e-2, abs32=1e-4)
    # what the slots hold at the end: the matrices (a column is contiguous) and the convolution's last inputs
    for s in (1, 2):
        S, tail = wants[s][1]
        held = state[slots[s]].cpu().double()
        close(held[: H * V * D].view(H, V, D), S.transpose(1, 2), "float32", f"state of sequence {s}", abs32=1e-4)
        if taps > 1:
            close(held[H * V * D:].view(taps - 1, -1), tail, "float32", f"convolution tail of sequence {s}", abs32=0.0)
    return got


# ---- whole models ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("senadra_gpu")
    return {name: write_case(root, name) for name in CONFIGS}


LENGTHS = {"P": [1, 9, 40, 75, 130], "Q": [3, 35, 70, 20, 100], "R": [2, 90, 33, 150], "S": [70, 5, 120, 33], "T": [41, 3, 77]}
_plain_cache = {}


def rounded_plain(folder, reqs, dtype):
    """The plain implementation with the input and the result of every matrix product rounded to ``dtype``: how far
    rounding alone moves the logits at each position."""
    cfg, w = plain.load_folder(folder)
    plain.product_rounding = lambda z: z.to(DT[dtype]).to(F64)
    try:
        return {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    finally:
        plain.product_rounding = None


def requests_and_plain(folders, name, lengths=None, seed=40, folder=None, reqs=None):
    key = (folder or name, tuple(lengths or LENGTHS[name]), seed)
    if key not in _plain_cache:
        if reqs is None:
            reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}
        want = plain_logits(folder or folders[name], reqs)
        rough = {dt: rounded_plain(folder or folders[name], reqs, dt) for dt in DT}
        _plain_cache[key] = (reqs, (want, rough))
    return _plain_cache[key]


def run_trace(folder, name, dtype, reqs, want_rough, steps, max_tokens, what, max_requests=4):
    from iian_b200.engine.replay import TraceReplayer
    want, rough = want_rough
    rp = TraceReplayer.from_folder(folder, dtype, max_tokens, BLOCK_SIZE[name], max_requests)
    got = replay_and_collect(rp, steps)
    rp.runner.check_device_status()
    rp.runner.manager.check_invariants()
    assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(len(t) for t in reqs.values())
    scale = max(w.abs().max().item() for w in want.values())
    floor = 3e-5 * max(1.0, scale) if dtype == "float32" else 3e-2 * scale
    over = []
    for (rid, pos) in sorted(got):
        e = (got[(rid, pos)].double() - want[rid][pos]).abs().max().item()
        tol = floor + 3.0 * (rough[dtype][rid][pos] - want[rid][pos]).abs().max().item()
        assert e <= 3.0 * tol, f"{name} {dtype} {what}: first wrong logits at {(rid, pos)}: {e:.3g} > 3 x {tol:.3g}; worst {max_error(got, want)}"
        if not e <= tol:
            over.append((rid, pos, e, tol))
    assert len(over) <= 0.02 * len(got), f"{name} {dtype} {what}: {len(over)} of {len(got)} positions beyond rounding, first {over[0]}"
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_stream_after_every_layer(folders, name, dtype):
    """The float32 stream behind every layer of a 50-token prompt: the first layer that differs names the mechanism."""
    from iian_b200.engine.replay import TraceReplayer
    cfg, w = plain.load_folder(folders[name])
    toks = random_tokens(CONFIGS[name]["vocab"], 50, 12)
    _, layers = plain.forward(cfg, w, toks, return_layers=True)
    rp = TraceReplayer.from_folder(folders[name], dtype, 64, BLOCK_SIZE[name], 4)
    seen = []
    for blk in rp.model.blocks:
        def wrapped(*a, _f=blk.forward, **k):
            r, d = _f(*a, **k)
            seen.append((r.clone(), None if d is None else d.clone()))
            return r, d
        blk.forward = wrapped
    rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": list(range(50))}], "end": ["a"]})
    assert len(seen) == len(cfg["layers"])
    for i, (r, d) in enumerate(seen):
        assert r.dtype == torch.float32, "the stream is kept in 32-bit"
        assert d is None, "a layer of this arrangement leaves nothing for the next one to add"
        ref = layers[i]
        # (in bfloat16 every layer adds rounding of its own on top of what it inherits; the 32-bit run is the sharp one)
        tol = (2e-5 if dtype == "float32" else 2e-2 * (i + 1)) * max(1.0, ref.abs().max().item())
        err = (r.double().cpu() - ref).abs().max().item()
        assert err <= tol, f"{name} {dtype}: stream behind layer {i} ({cfg['layers'][i]['type']}) off by {err:.3g} > {tol:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_under_every_cut(folders, name, dtype):
    reqs, want = requests_and_plain(folders, name)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    whole = run_trace(folders[name], name, dtype, reqs, want, trace_whole(reqs), rounded, "whole")
    for what, steps, cap, live in (("tail", trace_tail(reqs, 40), rounded, 4), ("portions", trace_portions(reqs), rounded, 4),
                                   ("mixed", trace_mixed(reqs, 2 * rounded, seed=1), 2 * rounded, 4),
                                   ("mixed, two slots", trace_mixed(reqs, rounded + 64, seed=2, max_live=2), rounded + 64, 2)):
        got = run_trace(folders[name], name, dtype, reqs, want, steps, cap, what, live)
        if dtype == "float32":      # every sum has an order fixed by the token's own position: the cut changes no bit
            worst = max((got[k] - whole[k]).abs().max().item() for k in got)
            assert worst <= 2e-6, f"{name} {what}: differs from the whole prompt by {worst}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_two_tokens_over_chunk_edges(folders, dtype):
    """Chunks of 24 and 17 positions under pages of 16: portions of two tokens, single tokens and portions of five walk over
    every edge; the recurrences go from step to step through their slot."""
    toks = random_tokens(211, 60, 8)
    reqs, want = requests_and_plain(folders, "P", reqs={"a": toks}, seed=8, lengths=[60])
    for size in (2, 1, 5):
        steps = [{"step": i, "entries": [{"id": "a", "tokens": toks[p:p + size], "want": list(range(len(toks[p:p + size])))}],
                  "end": ["a"] if p + size >= 60 else []} for i, p in enumerate(range(0, 60, size))]
        run_trace(folders["P"], "P", dtype, reqs, want, steps, 64, f"portions of {size}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_far_token(folders, dtype):
    """200 tokens decoded one by one behind a short prompt (chunk edges pass under decoded tokens, the recurrences run on),
    and a token whose embedding is large, met once early and again at the end: the layer without a chunk and the
    recurrences carry it."""
    reqs, want = requests_and_plain(folders, "P", [230], seed=90)
    run_trace(folders["P"], "P", dtype, reqs, want, trace_tail(reqs, 200), 256, "long decoding")
    reqs, want = requests_and_plain(folders, "R", [200], seed=91)
    run_trace(folders["R"], "R", dtype, reqs, want, trace_tail(reqs, 190), 256, "long decoding")
    d = folders["R"] + "_far"
    if not os.path.isdir(d):
        cfg, w = plain.load_folder(folders["R"])
        from iian_b200.weights.safetensors_io import write_safetensors
        w = {k: (v.float() if v.is_floating_point() else v) for k, v in w.items()}
        w["embed"][7] *= 6.0
        os.makedirs(d)
        write_safetensors(os.path.join(d, "model.safetensors"), {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in w.items()})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
    toks = [t if t != 7 else 8 for t in random_tokens(97, 400, 3)]
    toks[4] = toks[-1] = toks[-30] = 7
    reqs, want = requests_and_plain(folders, "R", folder=d, reqs={"far": toks})
    run_trace(d, "R", dtype, reqs, want, trace_whole(reqs), 448, "far token, whole")
    run_trace(d, "R", dtype, reqs, want, trace_tail(reqs, 40), 448, "far token, decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    name = "Q"
    cfg, w = plain.load_folder(folders[name])
    prompts = [random_tokens(300, n, 70 + i) for i, n in enumerate([1, 6, 30, 50, 77])]
    want = []
    for p in prompts:
        toks, margins = list(p), []
        for _ in range(10):
            row = plain.forward(cfg, w, toks)[-1]
            top = torch.topk(row, 2).values
            margins.append((top[0] - top[1]).item())
            toks.append(int(torch.argmax(row)))
        want.append((toks[len(p):], margins))
    for kw in (dict(budget=1024, kv_cache_tokens=1024, cuda_graphs=True), dict(budget=13, kv_cache_tokens=1024, cuda_graphs=True),
               dict(budget=64, kv_cache_tokens=128, cuda_graphs=False)):
        sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget"), max_num_seqs=8)
        eng = Engine(folders[name], EngineConfig(dtype=dtype, block_size=BLOCK_SIZE[name], sched=sched, max_model_len=128, **kw))
        got = eng.generate(prompts, max_tokens=10, temperature=0.0)
        for g, (wt, margins) in zip(got, want):
            for k, (a, b) in enumerate(zip(g, wt)):
                if a != b:
                    assert dtype == "bfloat16" and margins[k] < 0.05, f"{kw}: token {k}: {g} vs {wt} (margin {margins[k]:.4f})"
                    break
        if kw.get("cuda_graphs"):
            assert eng.runner.num_graphs >= 1
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_trace_runner_as_a_program(folders, tmp_path):
    reqs, (want, _) = requests_and_plain(folders, "R")
    steps = trace_mixed(reqs, 384, seed=4)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["R"], "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "384", "--block-size", "32"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    fed = {}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, 97)
        r = 0
        for ent in s["entries"]:
            for k in ent["want"]:
                p = fed.get(ent["id"], 0) + k
                assert np.abs(rows[r] - want[ent["id"]][p].numpy()).max() < 1e-4
                r += 1
            fed[ent["id"]] = fed.get(ent["id"], 0) + len(ent["tokens"])
