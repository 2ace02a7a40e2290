"""Nogelorn on the GPU.  Each new kernel alone against the plain functions of tests/plain_nogelorn.py (the normalised addend
with the next norm; rotation with rescaled frequencies and a magnitude, the unit norm behind it and the cache write;
attention with a stand-out key just inside and just outside the window, among the kept first keys and right behind them, at
page borders and far away, as rows of a portion and as decoded tokens, with a sink and a gate per head, through the general
kernel and through the tensor-core kernels; the decayed scan in every lane form, both kinds of decay, cut into steps, with
slots used again; the router's softmax over the chosen logits with the shared expert); then whole models under every way of
cutting the work, in 32-bit and in bfloat16; greedy generation through the engine's entry point with and without CUDA
graphs; the trace runner as a program."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from helpers import max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
import plain_nogelorn as plain
from nogelorn_cases import BLOCK_SIZE, CONFIGS, plain_logits, rounded_plain, router_margins, write_case

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
@pytest.mark.parametrize("h", [72, 100, 1000, 4100, 30])
def test_normalised_addend_and_the_next_norm(dtype, h):
    g = torch.Generator().manual_seed(h)
    x = torch.randn(5, h, generator=g) * 3
    y = (torch.randn(5, h, generator=g) * 7).to(DT[dtype])
    e = torch.randn(5, h, generator=g)
    u, w = torch.randn(h, generator=g) * 0.2, torch.randn(h, generator=g) * 0.2
    for with_u, with_e, with_out, with_y in ((True, False, True, True), (True, True, True, True), (False, False, True, True),
                                             (True, False, False, True), (False, True, True, False)):
        res = x.to(DEV).clone()
        out = torch.empty(5, h, device=DEV, dtype=DT[dtype]) if with_out else None
        K().normed_add_rms_norm(res, y.to(DEV) if with_y else None, (u + 1.0).to(DEV) if with_u else None, 1e-5,
                                e.to(DEV) if with_e else None, (w + 1.0).to(DEV) if with_out else None, 1e-6, out)
        s = x.double()
        if with_y:
            s = s + (plain.offset_rms_norm(y.double(), u.double(), 1e-5) if with_u else y.double())
        if with_e:
            s = s + e.double()
        close(res, s, "float32", f"stream after the normalised addend, width {h}")
        if with_out:
            close(out, plain.offset_rms_norm(s, w.double(), 1e-6), dtype, f"the next norm, width {h}", rel16=8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weighted_sum_and_heads_norm_with_either_gate(dtype):
    g = torch.Generator().manual_seed(2)
    a, b = torch.randn(7, 96, generator=g).to(DT[dtype]), torch.randn(7, 96, generator=g).to(DT[dtype])
    out = torch.empty(7, 96, dtype=DT[dtype], device=DEV)
    K().weighted_sum2(a.to(DEV), 0.7, b.to(DEV), 1.3, out)
    close(out, 0.7 * a.double() + 1.3 * b.double(), dtype, "weighted sum of two", rel16=8e-3)
    for heads, dv, act in ((1, 120, "sigmoid"), (3, 40, "silu"), (5, 12, "silu"), (2, 128, "sigmoid"), (1, 2048, "sigmoid"), (2, 1100, "silu")):
        x = torch.randn(6, heads * dv, generator=g) * 4
        w = torch.randn(heads * dv, generator=g)
        wide = torch.randn(6, heads * dv + 8, generator=g).to(DT[dtype])
        out = torch.empty(6, heads * dv, dtype=DT[dtype], device=DEV)
        K().head_norm_gate_act(x.to(DEV), w.to(DEV), wide.to(DEV)[:, 8:], out, num_heads=heads, eps=1e-5, gate_act=act)
        z = wide[:, 8:].double()
        want = (plain.unit_rms(x.double().view(6, heads, dv), 1e-5).reshape(6, -1) * w.double()) * (torch.sigmoid(z) if act == "sigmoid" else plain.silu(z))
        close(out, want, dtype, f"{heads} heads of {dv}, {act} gate", rel16=1e-2)


# ---- rotation, unit norm, cache write ------------------------------------------------------------------------
def _fill_cache(dtype, nh, nkv, dk, dv, freqs, magnitude, unit, positions, page, seed, eps=1e-5, gate_cols=0, boost=None):
    """Projections of len(positions) tokens of one sequence through the kernels into a paged cache; returns what the plain
    functions make of the same rows."""
    g = torch.Generator().manual_seed(seed)
    n = len(positions)
    width = nh * dk + nkv * dk + nkv * dv + gate_cols
    proj = torch.randn(n, width + 8, generator=g).to(DT[dtype])            # the mixer's columns start behind 8 others
    n_pages = -(-(max(positions) + 1) // page) + 3
    order = torch.randperm(n_pages, generator=g)[: -(-(max(positions) + 1) // page)].to(torch.int32)       # scattered pages
    kc = torch.zeros(n_pages, nkv, page, dk, dtype=DT[dtype], device=DEV)
    vc = torch.zeros(n_pages, nkv, page, dv, dtype=DT[dtype], device=DEV)
    pos = torch.tensor(positions, dtype=torch.int32)
    slots = (order[(pos // page).long()] * page + pos % page).to(torch.int32)
    q = torch.empty(n, nh, dk, dtype=DT[dtype], device=DEV)
    rot = 2 * freqs.numel() if freqs is not None else 0
    table = None
    if rot:
        table = torch.empty(n, rot // 2, 2, device=DEV)
        K().rotary_table_scaled(freqs.to(DEV), pos.to(DEV), rot // 2, magnitude, table)
    cols = proj.to(DEV)[:, 8:]
    K().rotate_unit_store(cols, 0, nh * dk, (nh + nkv) * dk, q, kc, vc, table, slots.to(DEV), num_heads=nh, num_kv_heads=nkv, k_dim=dk,
                          v_dim=dv, rot_dim=rot, eps=eps, unit_norm=unit)
    p64 = proj.double()[:, 8:]
    qw = p64[:, : nh * dk].reshape(n, nh, dk)
    kw = p64[:, nh * dk:(nh + nkv) * dk].reshape(n, nkv, dk)
    if rot:
        qw, kw = plain.rotate_half(qw, pos, freqs, magnitude), plain.rotate_half(kw, pos, freqs, magnitude)
    if unit:
        qw, kw = plain.unit_rms(qw, eps), plain.unit_rms(kw, eps)
    v0 = (nh + nkv) * dk
    return SimpleNamespace(proj=proj, cols=cols, q=q, kc=kc, vc=vc, order=order, slots=slots, pos=pos, q_want=qw, k_want=kw,
                           v_want=p64[:, v0: v0 + nkv * dv].reshape(n, nkv, dv), gate=p64[:, v0 + nkv * dv:], gate_off=v0 + nkv * dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, dk, dv, rot, unit, kind", [(6, 2, 16, 24, 8, True, "bands"), (3, 3, 40, 24, 40, False, "ramp"),
                                                              (2, 1, 128, 128, 0, True, None), (8, 2, 64, 64, 32, True, None),
                                                              (1, 1, 200, 8, 100, False, "ramp")])
def test_rotation_unit_norm_and_cache_write(dtype, nh, nkv, dk, dv, rot, unit, kind):
    page = 8
    positions = [0, 1, 7, 8, 9, 70000][: 6 if rot else 5]                     # a far position: the angle is a float64 product
    freqs, mag = None, 1.0
    if rot:
        freqs = plain.base_frequencies(rot, 777.0)
        if kind == "bands":
            freqs = plain.banded_frequencies(rot, 777.0, 8.0, 1.0, 4.0, 64.0)
        elif kind == "ramp":
            freqs, mag = plain.ramped_frequencies(rot, 777.0, 4.0, 40.0, 16.0, 1.0)
    c = _fill_cache(dtype, nh, nkv, dk, dv, freqs, mag, unit, positions, page, seed=dk)
    close(c.q, c.q_want, dtype, "rotated, normalised queries", rel16=1e-2)
    cells = c.slots.long()
    k_got = c.kc.permute(0, 2, 1, 3).reshape(-1, nkv, dk)[cells.to(DEV)]
    v_got = c.vc.permute(0, 2, 1, 3).reshape(-1, nkv, dv)[cells.to(DEV)]
    close(k_got, c.k_want, dtype, "keys in their cells", rel16=1e-2)
    assert torch.equal(v_got.cpu().double(), c.v_want), "the values go into their cells exactly as projected"
    assert int((c.kc != 0).any(-1).any(1).sum()) == len(positions), "cells of other tokens were written"
    if rot and unit:      # the order matters: a norm BEFORE the rotation gives something else where only part of the head turns
        other = plain.rotate_half(plain.unit_rms(c.proj.double()[:, 8: 8 + nh * dk].reshape(-1, nh, dk), 1e-5), c.pos, freqs, mag)
        assert rot == dk or mag == 1.0 or (other - c.q_want).abs().max() > 1e-3


def test_the_positions_table_follows_the_plug_ins_frequencies():
    """The product's own frequency formulas (parts/position.py) against the plain ones, and the table kernel at a far position."""
    from iian_b200.config.spec import PartSpec
    from iian_b200.parts.position import ScaledRotary
    for dims, base, sc, want in (
            (64, 30000.0, dict(kind="bands", factor=8.0, low=1.0, high=4.0, original=256), plain.banded_frequencies(64, 30000.0, 8.0, 1.0, 4.0, 256)),
            (48, 1e6, dict(kind="ramp", factor=4.0, original=512, fast=32.0, slow=1.0), plain.ramped_frequencies(48, 1e6, 4.0, 512, 32.0, 1.0))):
        part = ScaledRotary(PartSpec("scaled_rotary", {"dim": dims, "base": base, "scaling": sc}), torch.float32, DEV)
        f, m = want if isinstance(want, tuple) else (want, 1.0)
        assert (part.inv_freq64.cpu() - f).abs().max() < 1e-15 and part.magnitude == pytest.approx(m)
        pos = torch.tensor([0, 3, 123456], dtype=torch.int32, device=DEV)
        table = torch.empty(3, dims // 2, 2, device=DEV)
        K().rotary_table_scaled(part.inv_freq64, pos, dims // 2, part.magnitude, table)
        ang = pos.cpu().double()[:, None] * f[None, :]
        assert (table[..., 0].cpu().double() - torch.cos(ang) * m).abs().max() < 2e-7
        assert (table[..., 1].cpu().double() - torch.sin(ang) * m).abs().max() < 2e-7


# ---- attention ---------------------------------------------------------------------------------------------
def _plain_attention(c, nh, nkv, dv, scale, window, keep, sink, gate):
    n = c.q_want.shape[0]
    o = plain.masked_attention(c.q_want, c.k_want, c.v_want, scale, window, keep, sink=sink)
    if gate is not None:
        o = o * torch.sigmoid(gate)[:, :, None]
    group = torch.arange(nh) // (nh // nkv)
    see = plain.visibility(c.pos, n, window, keep)
    s = (torch.einsum("ihd,jhd->hij", c.q_want, c.k_want[:, group]) * scale).masked_fill(~see[None], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink[:, None, None].expand(nh, n, 1)], dim=-1)
    return o.reshape(n, nh * dv), torch.softmax(s, -1)[..., :n]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, dk, dv, window, keep, page", [
    (6, 2, 16, 24, 37, 5, 16), (4, 4, 64, 64, 33, 0, 8), (8, 2, 64, 64, 64, 0, 16), (2, 1, 128, 128, None, 0, 32), (3, 1, 24, 8, 5, 9, 16),
    (4, 2, 128, 128, 150, 0, 16), (4, 2, 128, 128, 150, 40, 16), (2, 2, 96, 96, 100, 33, 16), (4, 1, 64, 32, 48, 16, 8),
    (8, 2, 64, 64, 64, 70, 16), (4, 2, 128, 128, 150, 200, 16), (8, 1, 128, 128, 40, 129, 32)])
def test_attention_sees_window_kept_keys_and_sink_exactly(dtype, nh, nkv, dk, dv, window, keep, page):
    _attention_case(dtype, nh, nkv, dk, dv, window, keep, page, 300 if window else 1500)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, dk, dv, window, keep, page, n", [
    (8, 4, 64, 64, 136, 20, 16, 1400), (8, 2, 128, 128, 700, 200, 16, 2600), (4, 4, 128, 128, 96, 0, 16, 1200), (6, 2, 96, 96, 136, 20, 16, 1100),
    (4, 2, 128, 128, 1024, 64, 16, 3000)])
def test_attention_in_long_contexts(dtype, nh, nkv, dk, dv, window, keep, page, n):
    """The same far behind the window: many key tiles are skipped between the kept keys and the window, decoded tokens split
    their keys into parts, long portions run on the tcgen05 kernel."""
    _attention_case(dtype, nh, nkv, dk, dv, window, keep, page, n)


def _attention_case(dtype, nh, nkv, dk, dv, window, keep, page, n):
    """Keys are made to stand out by putting a multiple of a query into their cache cells: one just inside and one just outside
    the last token's window, one that is the last kept key and one right behind the kept keys (without a window: one at
    position 1, hundreds of tokens back).  Queries: a portion of the last 7 tokens, the same tokens one by one, the first ones,
    long portions.  Heads of 64 / 128 with equal sizes run on the tensor-core kernels in bfloat16 (kept keys, sink and gate inside
    them)."""
    w = window or n                             # without a window: enough keys that decoding cuts them into several parts
    inside, outside = (max(n - w, 1), n - w - 1) if window else (1, -1)
    c = _fill_cache(dtype, nh, nkv, dk, dv, plain.base_frequencies(min(dk, 16) // 2 * 2, 777.0), 1.0, True, list(range(n)), page,
                    seed=nh * dk, gate_cols=nh)
    first_of_group = torch.arange(nkv) * (nh // nkv)
    marks = [(inside, n - 1), (outside, n - 2)]
    if keep and outside > keep:
        marks += [(keep - 1, n - 3), (keep, n - 4)]
    for j, asker in marks:
        if j < 0:
            continue
        key = (1.5 * c.q_want[asker, first_of_group]).to(DT[dtype])                       # [nkv, dk]
        cell = int(c.slots[j])
        c.kc[cell // page, :, cell % page, :] = key.to(DEV)
        c.k_want[j] = key.double()
    sink = torch.randn(nh, generator=torch.Generator().manual_seed(5)) * 2
    scale = 4.0 / dk
    want, p = _plain_attention(c, nh, nkv, dv, scale, window, keep, sink.double(), c.gate)
    assert p[:, n - 1, inside].max() > 0.2, "the stand-out key inside the window must matter"
    if outside >= keep:
        assert p[:, n - 1, outside].max() == 0 and p[:, n - 2, outside].max() > 0.2     # one token earlier it was still seen
    elif outside >= 0:
        assert p[:, n - 2, outside].max() > 0.2 and p[:, n - 1, outside].max() > 0      # behind the window, but a kept key
    if len(marks) == 4:
        assert p[:, n - 3, keep - 1].max() > 0.2 and p[:, n - 4, keep].max() == 0       # the last kept key; the first forgotten one
    bt = torch.full((1, max(64, c.order.numel())), -1, dtype=torch.int32)
    bt[0, : c.order.numel()] = c.order
    gate = c.cols[:, c.gate_off: c.gate_off + nh]
    from iian_b200.ops import cuda_backend
    before = dict(cuda_backend.LAUNCHES_BY_ENTRY)
    for rows in (list(range(n - 7, n)), [n - 4], [n - 3], [n - 2], [n - 1], list(range(0, 3)), list(range(n - 200, n)), list(range(0, 130)),
                 list(range(keep, keep + 2)) if keep else [0]):
        r = torch.tensor(rows)
        meta = SimpleNamespace(positions=c.pos[r].to(DEV), seq_of_token=torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                               cu_q=torch.tensor([0, len(rows)], dtype=torch.int32, device=DEV),
                               ctx_len=torch.tensor([rows[-1] + 1], dtype=torch.int32, device=DEV), block_table=bt.to(DEV),
                               slots=c.slots[r].to(DEV), num_seqs=1, num_tokens=len(rows), max_q_len=len(rows), max_ctx=rows[-1] + 1,
                               decode_only=len(rows) == 1, h_q_len=[len(rows)], h_ctx_len=[rows[-1] + 1])
        out = torch.empty(len(rows), nh * dv, dtype=DT[dtype], device=DEV)
        K().window_attention(c.q[r.to(DEV)].reshape(len(rows), nh * dk), c.kc, c.vc, out, meta, num_heads=nh, num_kv_heads=nkv, k_dim=dk,
                             v_dim=dv, scale=scale, window=window, keep_first=keep, sink=sink.to(DEV), gate=gate[r.to(DEV)],
                             gate_per_head=True)
        close(out, want[r], dtype, f"attention rows {rows[0]}..{rows[-1]}", rel16=2.5e-2)
    K().check_device_status()
    fast = dtype == "bfloat16" and dk == dv and dk in (64, 128)
    ran = {k: v - before.get(k, 0) for k, v in cuda_backend.LAUNCHES_BY_ENTRY.items() if v != before.get(k, 0)}
    assert ("window_attention" not in ran) == fast, f"which kernel served it: {ran}"
    # without the sink the first tokens come out differently: it is in the denominator
    no_sink, _ = _plain_attention(c, nh, nkv, dv, scale, window, keep, None, c.gate)
    assert (no_sink[:3] - want[:3]).abs().max() > 1e-3


# ---- the decayed scan ---------------------------------------------------------------------------------------
def _plain_scan(proj, H, d, dv, act, q_scale, head_decay, z, bias, tau, state=None):
    n = proj.shape[0]
    f = plain.silu if act else (lambda t: t)
    q = f(proj[:, : H * d]).view(n, H, d) * q_scale
    k = f(proj[:, H * d: 2 * H * d]).view(n, H, d)
    v = f(proj[:, 2 * H * d: 2 * H * d + H * dv]).view(n, H, dv)
    if head_decay is not None:
        a = head_decay[None, :, None].expand(n, H, d)
    else:
        a = torch.exp(torch.nn.functional.logsigmoid(z + bias) / tau).view(n, H, d)
    o, S = plain.decayed_outer_scan(q, k, v, a, state)
    return o.reshape(n, H * dv), S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, d, dv, per_channel", [(3, 24, 40, False), (2, 16, 24, True), (4, 32, 32, False), (1, 160, 16, True), (1, 8, 8, True),
                                                   (2, 64, 128, False), (1, 300, 6, True), (5, 128, 48, True), (2, 48, 64, True), (1, 512, 20, False)])
def test_decayed_scan_cut_into_steps_with_slots_used_again(dtype, H, d, dv, per_channel):
    """Three sequences of unequal length walked in steps of 1 to 29 tokens beside each other, against the plain recurrence over
    whole sequences; then a new sequence in a slot that was used (zeroed by the storage, as at admission)."""
    g = torch.Generator().manual_seed(H * d + dv)
    lengths = [37, 5, 64]
    width = 2 * H * d + H * dv
    projs = [(torch.randn(n, width + 4, generator=g) * 0.7).to(DT[dtype]) for n in lengths]
    zs = [torch.randn(n, H * d, generator=g) * 2 for n in lengths]
    bias = torch.randn(H * d, generator=g)
    head_decay = torch.rand(H, generator=g) * 0.5 + 0.5
    tau, q_scale, act = 3.0, d ** -0.5, not per_channel
    want = [_plain_scan(p.double()[:, 4:], H, d, dv, act, q_scale, None if per_channel else head_decay.double(), z.double(), bias.double(), tau)[0]
            for p, z in zip(projs, zs)]
    state = torch.zeros(4, H, -(-dv // 16), 16, (d + 3) // 4 * 4, device=DEV)
    slots = [2, 0, 3]
    fed = [0, 0, 0]
    got = [torch.zeros(n, H * dv) for n in lengths]
    sizes = [1, 7, 2, 29, 1, 1, 16, 3, 17, 2]
    step = 0
    while any(f < n for f, n in zip(fed, lengths)):
        rows, cu, sl, take = [], [0], [], []
        for i, n in enumerate(lengths):
            c = min(sizes[(step + i) % len(sizes)], n - fed[i])
            if c <= 0 or (step + i) % 4 == 3:
                continue
            take.append((i, fed[i], c))
            cu.append(cu[-1] + c)
            sl.append(slots[i])
        step += 1
        if not take:
            continue
        # a padding sequence rides along: slot -1, its rows come out as zeros and no state is touched
        cu.append(cu[-1] + 1)
        sl.append(-1)
        proj = torch.cat([projs[i][a:a + c] for i, a, c in take] + [projs[0][:1]]).to(DEV)
        z = torch.cat([zs[i][a:a + c] for i, a, c in take] + [zs[0][:1]]).to(DEV)
        out = torch.full((proj.shape[0], H * dv), 7.0, device=DEV)
        K().decay_scan(proj[:, 4:], 0, H * d, 2 * H * d, state, torch.tensor(cu, dtype=torch.int32, device=DEV),
                       torch.tensor(sl, dtype=torch.int32, device=DEV), out, num_heads=H, dim=d, v_dim=dv,
                       activation="silu" if act else None, q_scale=q_scale, head_decay=None if per_channel else head_decay.to(DEV),
                       z=z if per_channel else None, z_bias=bias.to(DEV) if per_channel else None, tau=tau,
                       max_q_len=max(c for _, _, c in take))
        assert (out[-1] == 0).all()
        for k, (i, a, c) in enumerate(take):
            got[i][a:a + c] = out[cu[k]:cu[k + 1]].cpu()
            fed[i] += c
    for i in range(3):
        close(got[i], want[i], "float32", f"sequence {i} of {H} heads {d} x {dv}", abs32=3e-5)
    assert (state[1] == 0).all(), "a slot no sequence had was written"
    # slot 2 again, zeroed as the storage does at admission
    state[2].zero_()
    out = torch.empty(5, H * dv, device=DEV)
    K().decay_scan(projs[1].to(DEV)[:, 4:], 0, H * d, 2 * H * d, state, torch.tensor([0, 5], dtype=torch.int32, device=DEV),
                   torch.tensor([2], dtype=torch.int32, device=DEV), out, num_heads=H, dim=d, v_dim=dv, activation="silu" if act else None,
                   q_scale=q_scale, head_decay=None if per_channel else head_decay.to(DEV), z=zs[1].to(DEV) if per_channel else None,
                   z_bias=bias.to(DEV) if per_channel else None, tau=tau, max_q_len=5)
    close(out, want[1], "float32", "a sequence in a slot that was used before", abs32=3e-5)


# ---- experts: softmax over the chosen logits, an expert every token uses ---------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, experts, top, width, ff, shared", [(1, 3, 1, 64, 32, 16), (9, 5, 2, 96, 48, 0), (300, 8, 3, 128, 64, 96),
                                                                (40, 2, 2, 100, 36, 20), (17, 12, 4, 64, 24, 40)])
def test_softmax_routed_experts_with_a_shared_expert(dtype, n, experts, top, width, ff, shared):
    from iian_b200.config.spec import PartSpec
    from iian_b200.engine.runner import StepContext, Workspace
    from iian_b200.parts.experts import RoutedExperts
    g = torch.Generator().manual_seed(n + experts)
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "num_experts": experts, "top": top, "intermediate_size": ff,
                                                     "activation": "silu", "score": "softmax_top", "weight_on": "output",
                                                     "shared_intermediate_size": shared}), DT[dtype], torch.device(DEV))
    tensors = {name: (torch.randn(*ts.shape, generator=g) * (1.0 if name.startswith("router") else 0.15)).to(DT[dtype])
               for name, ts in part.tensors().items()}
    part.bind({k: v.to(DEV) for k, v in tensors.items()})
    h = torch.randn(n, width, generator=g).to(DT[dtype])
    ctx = StepContext(Workspace(torch.device(DEV)))
    out = part.forward(h.to(DEV), ctx)
    w64 = {k: v.double() for k, v in tensors.items()}
    cfg = {"router": {"top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.experts_feed_forward(cfg, w64, "", h.double())
    ids, _ = plain.router_choice(h.double(), w64, "", top)
    z = h.double() @ w64["router"].T + w64["router.b"]
    srt = torch.sort(z, dim=-1, descending=True).values
    safe = (srt[:, top - 1] - srt[:, top]).abs() > (1e-4 if dtype == "float32" else 0.1) if top < experts else torch.ones(n, dtype=torch.bool)
    assert safe.sum() > 0.6 * n                    # rows where rounding cannot change the choice
    close(out[safe.to(DEV)], want[safe], dtype, "experts' weighted sum plus the shared expert", rel16=3e-2, abs32=3e-5)


# ---- whole models --------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("nogelorn_gpu")
    out = {(name, "float32"): write_case(root, name) for name in CONFIGS}
    out.update({(name, "bfloat16"): write_case(root, name, router_step=3.0) for name in CONFIGS})     # see spread_router_biases
    return out


LENGTHS = {"G": [1, 9, 40, 75, 130], "H": [3, 35, 70, 20, 100], "I": [2, 90, 33, 150], "J": [70, 5, 120, 33], "Q": [41, 3, 77]}
_plain_cache = {}


def requests_and_plain(folders, name, dtype, lengths=None, seed=40, folder=None, reqs=None):
    folder = folder or folders[(name, dtype)]
    key = (folder, tuple(lengths or LENGTHS[name]), seed)
    if key not in _plain_cache:
        if reqs is None:
            reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}
        _plain_cache[key] = (reqs, (plain_logits(folder, reqs), {dtype: rounded_plain(folder, reqs, DT[dtype])}, router_margins(folder, reqs)))
    return _plain_cache[key]


def run_trace(folder, name, dtype, reqs, want_rough, steps, max_tokens, what, max_requests=4):
    from iian_b200.engine.replay import TraceReplayer
    want, rough, margins = want_rough
    rp = TraceReplayer.from_folder(folder, dtype, max_tokens, BLOCK_SIZE[name], max_requests)
    got = replay_and_collect(rp, steps)
    rp.runner.check_device_status()
    rp.runner.manager.check_invariants()
    assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(len(t) for t in reqs.values())
    scale = max(w.abs().max().item() for w in want.values())
    floor = 3e-5 * max(1.0, scale) if dtype == "float32" else 3e-2 * scale
    over = []
    # a router whose choice hangs on less than the rounding of its logits may choose otherwise in bfloat16; that token's
    # feed-forward output is then another (normalised, so never small).  Such positions are not compared.
    hair = 0.0 if dtype == "float32" else 0.06
    skipped = 0
    for (rid, pos) in sorted(got):
        assert torch.isfinite(got[(rid, pos)]).all()
        if margins[rid][pos] < hair:
            skipped += 1
            continue
        e = (got[(rid, pos)].double() - want[rid][pos]).abs().max().item()
        tol = floor + 3.0 * (rough[dtype][rid][pos] - want[rid][pos]).abs().max().item()
        assert e <= 3.0 * tol, f"{name} {dtype} {what}: first wrong logits at {(rid, pos)}: {e:.3g} > 3 x {tol:.3g}; worst {max_error(got, want)}"
        if not e <= tol:
            over.append((rid, pos, e, tol))
    # the rounded oracle is ONE draw of the rounding noise at a touchy position: a few positions may be further off than it
    assert skipped <= 0.15 * len(got), f"{name}: {skipped} of {len(got)} positions have a router on a hair"
    assert len(over) <= 0.02 * len(got), f"{name} {dtype} {what}: {len(over)} of {len(got)} positions beyond rounding, first {over[0]}"
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_under_every_cut(folders, name, dtype):
    reqs, want = requests_and_plain(folders, name, dtype)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    folder = folders[(name, dtype)]
    whole = run_trace(folder, name, dtype, reqs, want, trace_whole(reqs), rounded, "whole")
    for what, steps, cap, live in (("tail", trace_tail(reqs, 40), rounded, 4), ("portions", trace_portions(reqs), rounded, 4),
                                   ("mixed", trace_mixed(reqs, 2 * rounded, seed=1), 2 * rounded, 4),
                                   ("mixed, two slots", trace_mixed(reqs, rounded + 64, seed=2, max_live=2), rounded + 64, 2)):
        got = run_trace(folder, name, dtype, reqs, want, steps, cap, what, live)
        if dtype == "float32":      # every sum has an order fixed by the token's own position: the cut changes no bit
            worst = max((got[k] - whole[k]).abs().max().item() for k in got)
            assert worst <= 2e-6, f"{name} {what}: differs from the whole prompt by {worst}"


def test_the_stream_after_every_layer_run(folders):
    """The float32 residual stream after each layer run against the plain implementation's (what a layer still owes to the
    stream is added here by hand)."""
    from iian_b200.engine.replay import TraceReplayer
    toks = random_tokens(211, 21, 3)
    cfg, w = plain.load_folder(folders[("G", "float32")])
    _, streams = plain.forward(cfg, w, toks, return_layers=True)
    rp = TraceReplayer.from_folder(folders[("G", "float32")], "float32", 64, 16, 2)
    seen = []

    def spy(fn):
        def run(residual, delta, ctx, cache, writes_cache, select_rows):
            res, owed = fn(residual, delta, ctx, cache, writes_cache, select_rows)
            y = owed.y.double()
            seen.append((res.double() + y / torch.sqrt((y * y).mean(-1, keepdim=True) + owed.eps) * owed.weight.double()).cpu())
            return res, owed
        return run
    for b in rp.model.blocks:
        b.forward = spy(b.forward)
    rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": list(range(21))}], "end": ["a"]})
    assert len(seen) == streams.shape[0] == 6
    for i, x in enumerate(seen):
        assert (x - streams[i]).abs().max() < 3e-5 * max(1.0, streams[i].abs().max().item()), f"layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_far_key(folders, dtype):
    """200 tokens decoded one by one behind a short prompt (windows pass over decoded tokens, the kept keys stay, pages are
    given back on the way, the recurrences run on), and a token whose embedding is large, met once early and again at the end:
    the recurrences and the kept keys carry it."""
    reqs, want = requests_and_plain(folders, "G", dtype, [230], seed=90)
    run_trace(folders[("G", dtype)], "G", dtype, reqs, want, trace_tail(reqs, 200), 256, "long decoding")
    reqs, want = requests_and_plain(folders, "I", dtype, [200], seed=91)
    run_trace(folders[("I", dtype)], "I", dtype, reqs, want, trace_tail(reqs, 190), 256, "long decoding")
    for name, seed in (("J", 92), ("H", 93)):          # heads of 128 with kept keys, heads of 64 with a sink: the tensor-core kernels
        reqs, want = requests_and_plain(folders, name, dtype, [300, 270], seed=seed)
        run_trace(folders[(name, dtype)], name, dtype, reqs, want, trace_tail(reqs, 150), 320, "long decoding")
        run_trace(folders[(name, dtype)], name, dtype, reqs, want, trace_mixed(reqs, 640, seed=5), 640, "long, mixed")
    d = folders[("G", dtype)] + "_far"
    if not os.path.isdir(d):
        cfg, w = plain.load_folder(folders[("G", dtype)])
        from iian_b200.weights.safetensors_io import write_safetensors
        w = {k: (v.float() if v.is_floating_point() else v) for k, v in w.items()}
        w["embed"][7] *= 6.0
        os.makedirs(d)
        write_safetensors(os.path.join(d, "model.safetensors"), {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in w.items()})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
    toks = [t if t != 7 else 8 for t in random_tokens(211, 400, 3)]
    toks[4] = toks[-1] = toks[-30] = 7                      # position 4 is the last kept key of the attention layer
    reqs, want = requests_and_plain(folders, "G", dtype, folder=d, reqs={"far": toks})
    run_trace(d, "G", dtype, reqs, want, trace_whole(reqs), 448, "far key, whole")
    run_trace(d, "G", dtype, reqs, want, trace_tail(reqs, 40), 448, "far key, decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    name = "H"
    cfg, w = plain.load_folder(folders[(name, dtype)])
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
        eng = Engine(folders[(name, dtype)], EngineConfig(dtype=dtype, block_size=BLOCK_SIZE[name], sched=sched, max_model_len=128, **kw))
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
    reqs, (want, _, _) = requests_and_plain(folders, "I", "float32")
    steps = trace_mixed(reqs, 384, seed=4)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[("I", "float32")], "--dtype", "float32",
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
