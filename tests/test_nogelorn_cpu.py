"""Nogelorn without a GPU: the plain implementation's mechanisms on cases worked out by hand, the configuration reader, the
tensor names, and the engine's host side (K/V pages beside state slots in ONE layer, a stretch of layers run several times
with caches of its own per run, windows with and without kept keys, page and slot reuse, portions, mixed batches, the
scheduler's entry point) with the torch stand-in for the kernels against the plain implementation."""
import json
import math
import os

import pytest
import torch

from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
import plain_nogelorn as plain
from fake_kernels import FakeKernels
from iian_b200 import EngineConfig, SchedulerConfig, ops
from iian_b200.config.registry import get_architecture, load_model_config
from iian_b200.engine.engine import Engine
from iian_b200.engine.model import Model, declare_tensors
from iian_b200.engine.replay import TraceReplayer
from iian_b200.models.qwen3 import ConfigError
from iian_b200.parts.base import KVNeed, StateNeed, member_cache_id
from nogelorn_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case

F64 = torch.float64


# ---- the plain implementation's mechanisms ------------------------------------------------------------
def test_plain_norm_adds_one_to_the_weight():
    x = torch.tensor([[3.0, -4.0]], dtype=F64)
    got = plain.offset_rms_norm(x, torch.tensor([0.0, 0.5], dtype=F64), 0.0)
    rms = math.sqrt(12.5)
    assert torch.allclose(got, torch.tensor([[3 / rms, -4 / rms * 1.5]], dtype=F64))


def test_plain_rotation_pairs_halves_and_passes_the_rest():
    v = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], dtype=F64).view(1, 1, 6).repeat(2, 1, 1)
    f = plain.base_frequencies(4, 100.0)
    assert f.tolist() == pytest.approx([1.0, 0.1])
    out = plain.rotate_half(v, torch.tensor([0, 3]), f, 1.5)
    assert torch.allclose(out[0, 0, :4], 1.5 * v[0, 0, :4]) and out[0, 0, 4:].tolist() == [5.0, 6.0]   # position 0: the magnitude alone
    a0, a1 = 3.0, 0.3
    assert out[1, 0, 0].item() == pytest.approx(1.5 * (1 * math.cos(a0) - 3 * math.sin(a0)))           # pairs (0, 2) and (1, 3)
    assert out[1, 0, 2].item() == pytest.approx(1.5 * (3 * math.cos(a0) + 1 * math.sin(a0)))
    assert out[1, 0, 3].item() == pytest.approx(1.5 * (4 * math.cos(a1) + 2 * math.sin(a1)))
    assert out[1, 0, 4:].tolist() == [5.0, 6.0]


def test_plain_frequencies_by_bands_and_by_ramp():
    # wavelengths 2 pi, 20 pi, 200 pi, 2000 pi against original 1000: below 1000 / 4 stays, above 1000 / 1 is divided, between blends
    f = plain.banded_frequencies(8, 10000.0, 8.0, 1.0, 4.0, 1000.0)
    base = [1.0, 0.1, 0.01, 0.001]
    assert f[0].item() == pytest.approx(base[0]) and f[1].item() == pytest.approx(base[1])
    s = (1000.0 / (2 * math.pi / 0.01) - 1.0) / 3.0
    assert 0 < s < 1 and f[2].item() == pytest.approx((1 - s) * 0.01 / 8 + s * 0.01)
    assert f[3].item() == pytest.approx(0.001 / 8)
    # ramp: c(t) = 8 ln(64 / (2 pi t)) / (2 ln 10000); lo = floor(c(8)) = 0, hi = ceil(c(1)) = 2
    g, m = plain.ramped_frequencies(8, 10000.0, 4.0, 64.0, 8.0, 1.0)
    assert m == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert g.tolist() == pytest.approx([1.0, 0.1 * (0.5 / 4 + 0.5), 0.01 / 4, 0.001 / 4])


def test_plain_window_keeps_the_first_keys_and_the_sink_counts_once():
    see = plain.visibility(torch.tensor([7]), 10, 3, 2)
    assert see[0].tolist() == [True, True, False, False, False, True, True, True, False, False]
    assert plain.visibility(torch.tensor([1]), 4, 3, 2)[0].tolist() == [True, True, False, False]
    assert plain.visibility(torch.tensor([5]), 6, None)[0].all()
    q = torch.zeros(1, 1, 2, dtype=F64)
    k = torch.zeros(3, 1, 2, dtype=F64)
    v = torch.tensor([[[1.0]], [[2.0]], [[6.0]]], dtype=F64)
    o = plain.masked_attention(q, k, v, 1.0, None, sink=torch.tensor([math.log(3.0)], dtype=F64), q_pos0=2)
    assert o[0, 0, 0].item() == pytest.approx((1 + 2 + 6) / (3 + 3))                  # three keys of weight 1, a sink of weight 3


def test_plain_scan_first_steps_by_hand():
    """One head, two key channels, one value channel: the decay multiplies the ROWS of the state (key channels)."""
    q = torch.tensor([[[1.0, 1.0]], [[1.0, 0.0]]], dtype=F64)
    k = torch.tensor([[[2.0, 3.0]], [[1.0, 1.0]]], dtype=F64)
    v = torch.tensor([[[5.0]], [[7.0]]], dtype=F64)
    a = torch.tensor([[[0.5, 0.1]], [[0.5, 0.1]]], dtype=F64)
    o, S = plain.decayed_outer_scan(q, k, v, a)
    assert o[0, 0, 0].item() == pytest.approx(10 + 15)                               # S_1 = k_1 v_1: the first decay meets zeros
    assert S[0, :, 0].tolist() == pytest.approx([0.5 * 10 + 7, 0.1 * 15 + 7])
    assert o[1, 0, 0].item() == pytest.approx(12.0)
    o2, S2 = plain.decayed_outer_scan(q[1:], k[1:], v[1:], a[1:], state=torch.tensor([[[10.0], [15.0]]], dtype=F64))
    assert torch.allclose(o2[0], o[1]) and torch.allclose(S2, S)                     # a cut changes nothing


def test_plain_router_softmax_runs_over_the_chosen_logits_only():
    w = {"router": torch.eye(4, dtype=F64), "router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=F64)}
    h = torch.tensor([[1.0, 3.0, -3.0, 0.5]], dtype=F64)                              # logits 1, 3, 2, 0.5
    ids, wts = plain.router_choice(h, w, "", 2)
    assert ids.tolist() == [[1, 2]]
    assert wts[0].tolist() == pytest.approx([math.e / (1 + math.e), 1 / (1 + math.e)])


def test_plain_run_order_adds_the_embedding_before_every_pass_but_the_first():
    cfg = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 3}}
    assert plain.run_order(cfg) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert plain.run_order({"layers": [0, 1]}) == [(0, False), (1, False)]


# ---- configuration, names, caches ------------------------------------------------------------------------
def test_config_round_trip_and_registry():
    arch = get_architecture("Nogelorn")
    for name, raw in CONFIGS.items():
        c = arch.load_config(raw)
        assert arch.load_config(arch.config_to_dict(c)) == c, name
        spec = arch.build_spec(c)
        spec.validate()
        assert [call.layer for call in spec.order] == [i for i, _ in plain.run_order(raw)]
        assert [call.before is not None for call in spec.order] == [again for _, again in plain.run_order(raw)]
        assert len({call.cache for call in spec.order}) == len(spec.order)            # every run has a cache of its own


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "6 heads for 4"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("decay_rank"), "right.a1"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0), "tau"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=9), "takes 9 of 6"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=26), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "lacks 'slow'"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["loop"].update(stop=7), "loop runs layers"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_name_the_place(edit, text):
    raw = json.loads(json.dumps(CONFIGS["G"]))
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        get_architecture("Nogelorn").load_config(raw)


def test_tensor_names_and_cache_needs(tmp_path):
    arch = get_architecture("Nogelorn")
    names = declare_tensors(arch, arch.build_spec(arch.load_config(CONFIGS["G"])))
    for n in ("embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.g", "l0.mix.norm",
              "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e4.up", "l0.mlp.shared.down", "l1.mix.left.q", "l1.mix.left.o",
              "l1.mix.right.a1", "l1.mix.right.a2", "l1.mix.right.a2.b", "l1.mix.right.norm", "l1.mix.right.g", "l2.mix.sink",
              "l2.mix.g", "l2.mix.o", "l3.mlp.e3.down"):
        assert n in names, n
    for n in ("head", "l1.norm2", "l1.norm2b", "l1.mlp.router", "l2.mlp.shared.gate", "l0.mlp.e5.up", "l1.mix.left.sink", "l1.mix.left.g",
              "l0.mix.a1", "l0.mix.sink"):
        assert n not in names, n
    assert names["l0.mix.norm"].shape == (120,) and names["l1.mix.right.norm"].shape == (16,)      # all heads | one head's
    assert names["l2.mix.g"].shape == (4, 96) and names["l2.mix.sink"].shape == (4,) and names["l2.mix.o"].shape == (96, 64)
    assert names["l1.mix.right.a1"].shape == (12, 96) and names["l1.mix.right.a2"].shape == (72, 12)
    assert names["l1.mix.left.v"].shape == (48, 96) and names["l1.mix.left.o"].shape == (96, 144)
    d = write_case(tmp_path, "G", store_dtype=torch.float32)
    with ops.use_kernels(FakeKernels()):
        needs = Model.from_folder(d, "float32", "cpu").cache_needs()
    # run order 0 | 1 2 | 1 2 | 3: caches 0 .. 5; a side-by-side layer's members under ids of their own
    pair = [(member_cache_id(c, 0), member_cache_id(c, 1)) for c in (1, 3)]
    assert sorted(needs) == sorted([0, 2, 4, 5] + [m for p in pair for m in p])
    assert needs[pair[0][0]] == needs[pair[1][0]] == KVNeed(2, 16, 24, 24)             # a plain window gives pages back
    assert needs[2] == needs[4] == KVNeed(4, 24, None, 16)                             # kept first keys: every page stays
    assert needs[pair[0][1]] == StateNeed((3, 1, 16, 24), torch.float32)               # blocks of 16 columns: 16 -> 1, 40 -> 3
    assert needs[0] == StateNeed((3, 3, 16, 24), torch.float32)


def test_the_decay_rank_comes_from_the_tensor_when_the_file_is_silent(tmp_path):
    d = write_case(tmp_path, "Q", store_dtype=torch.float32)
    path = os.path.join(d, "config.json")
    raw = json.load(open(path))
    assert raw["layers"][2]["mixer"]["right"].pop("decay_rank") == 4
    json.dump(raw, open(path, "w"))
    arch, cfg = load_model_config(d)
    assert cfg.layers[2].mixer.right.rank == 4 and cfg == arch.load_config(CONFIGS["Q"])


# ---- the host side under every way of cutting the work -------------------------------------------------
@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("nogelorn")
    out = {}
    for name in CONFIGS:
        d = write_case(root, name, store_dtype=torch.float32)
        with ops.use_kernels(FakeKernels()):
            out[name] = (d, Model.from_folder(d, "float32", "cpu"))
    return out


LENGTHS = {"G": [1, 9, 40, 75], "H": [3, 35, 70, 20, 2], "I": [2, 90, 33], "J": [45, 5, 20], "Q": [41, 3, 30]}


def test_the_stream_after_every_layer_run(cases):
    """The residual stream the engine holds after each layer run is the plain implementation's (the addend a layer still owes
    is added here by hand: y / rms(y) * (1 + w))."""
    d, model = cases["G"]
    toks = random_tokens(211, 12, 3)
    cfg, w = plain.load_folder(d)
    _, streams = plain.forward(cfg, w, toks, return_layers=True)
    seen = []
    blocks = model.blocks
    originals = [b.forward for b in blocks]

    def spy(fn):
        def run(residual, delta, ctx, cache, writes_cache, select_rows):
            res, owed = fn(residual, delta, ctx, cache, writes_cache, select_rows)      # every row is wanted: nothing is gathered
            y = owed.y.double()
            seen.append(res.double() + y / torch.sqrt((y * y).mean(-1, keepdim=True) + owed.eps) * owed.weight.double())
            return res, owed
        return run
    try:
        for b, fn in zip(blocks, originals):
            b.forward = spy(fn)
        with ops.use_kernels(FakeKernels()):
            rp = TraceReplayer(model, 64, 16, 2, native=False)
            rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": list(range(12))}], "end": ["a"]})
    finally:
        for b in blocks:
            del b.forward
    assert len(seen) == streams.shape[0] == 6
    for i, x in enumerate(seen):
        assert (x - streams[i]).abs().max() < 1e-4, f"layer run {i}"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_matches_plain_under_every_cut(cases, name):
    d, model = cases[name]
    reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, 40 + i) for i, n in enumerate(LENGTHS[name])}
    want = plain_logits(d, reqs)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    for what, steps, cap in (("whole", trace_whole(reqs), rounded), ("tail", trace_tail(reqs, 20), rounded),
                             ("portions", trace_portions(reqs), rounded), ("mixed", trace_mixed(reqs, 2 * rounded, seed=3), 2 * rounded)):
        with ops.use_kernels(FakeKernels()):
            rp = TraceReplayer(model, cap, BLOCK_SIZE[name], 4, native=False)
            got = replay_and_collect(rp, steps)
        rp.runner.manager.check_invariants()
        assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
        assert len(got) == sum(len(t) for t in reqs.values())
        bad = first_bad(got, want, 2e-4)
        assert bad is None, f"{name} {what}: first wrong logits at {bad}; worst {max_error(got, want)}"


def test_a_slot_that_is_used_again_starts_from_zero(cases):
    """Two state slots, five requests one after another and side by side: a request that inherits a slot must not see what
    the one before left in it -- in a layer's own state and in the state of a side-by-side layer's member."""
    d, model = cases["G"]
    reqs = {f"r{i}": random_tokens(211, n, 90 + i) for i, n in enumerate([30, 12, 25, 7, 18])}
    want = plain_logits(d, reqs)
    steps = trace_mixed(reqs, 128, seed=1, max_live=2)
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 2, native=False)
        got = replay_and_collect(rp, steps)
    bad = first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong logits at {bad}"


def test_plain_windows_give_pages_back_and_kept_keys_hold_theirs(cases):
    d, model = cases["G"]
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 4, native=False)
        toks = random_tokens(211, 120, 5)
        for p in range(0, 120, 8):
            rp.run_step({"step": p, "entries": [{"id": "a", "tokens": toks[p:p + 8], "want": []}], "end": []})
    mgr = rp.runner.manager
    by_window = {g.window: mgr.pools[i] for i, g in enumerate(mgr.groups)}
    assert set(by_window) == {24, None}
    assert by_window[24].num_blocks - by_window[24].num_free <= 3                       # the window's pages only
    assert by_window[None].num_blocks - by_window[None].num_free == 8                   # 120 tokens in pages of 16


def test_greedy_generation_through_the_scheduler(cases):
    d, model = cases["H"]
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(300, n, 70 + i) for i, n in enumerate([1, 6, 30, 50])]

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(torch.argmax(plain.forward(cfg, w, toks)[-1])))
        return toks[len(prompt):]
    want = [greedy(p, 5) for p in prompts]
    for kw in (dict(budget=64, kv_cache_tokens=512), dict(budget=11, kv_cache_tokens=512),        # whole prompts; portions
               dict(budget=16, kv_cache_tokens=96, enable_prefix_caching=True)):                   # few pages: preemption
        sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget"), max_num_seqs=4)
        with ops.use_kernels(FakeKernels()):
            eng = Engine(model, EngineConfig(dtype="float32", block_size=8, warmup=False, sched=sched, max_model_len=96, **kw))
            assert not eng.runner.prefix_caching                   # a model with state cannot start behind a shared prefix
            assert eng.generate(prompts, max_tokens=5, temperature=0.0) == want
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_command_line_writes_and_loads_a_folder(tmp_path):
    """``iian random-weights`` from a Nogelorn config.json, then the folder through the loader (names, shapes, the plug-in)."""
    from iian_b200.cli.main import main as cli_main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["I"]))
    out = tmp_path / "model"
    assert cli_main(["random-weights", str(cfg_path), str(out), "--seed", "3"]) == 0
    arch, cfg = load_model_config(str(out))
    assert arch.name == "Nogelorn" and cfg == arch.load_config(CONFIGS["I"])
    with ops.use_kernels(FakeKernels()):
        model = Model.from_folder(str(out), "float32", "cpu")
        rp = TraceReplayer(model, 64, 16, 2, native=False)
        logits = rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]})
    want = plain.forward(*plain.load_folder(str(out)), [1, 2, 3])[-1]
    assert (logits[0].double() - want).abs().max() < 2e-4
