"""Senadra without a GPU: the plain implementation's mechanisms on cases worked out by hand, the configuration reader, the
tensor names, and the engine's host side (K/V pages whose values have a size of their own, a latent row cache and state
slots side by side, layers that read another layer's pages, chunks, page and slot reuse, portions, mixed batches, the
scheduler's entry point) with the torch stand-in for the kernels against the plain implementation."""
import json
import math

import pytest
import torch

import plain_senadra as plain
from fake_kernels import FakeKernels
from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from iian_b200 import EngineConfig, SchedulerConfig, ops
from iian_b200.config.registry import architecture_of, get_architecture
from iian_b200.engine.engine import Engine
from iian_b200.engine.model import Model, declare_tensors
from iian_b200.engine.replay import TraceReplayer
from iian_b200.models.qwen3 import ConfigError
from iian_b200.parts.base import KVNeed, RowNeed, StateNeed
from senadra_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case

F64 = torch.float64


def T(*v):
    return torch.tensor(v, dtype=F64)


# ---- the plain implementation's mechanisms ------------------------------------------------------------
def test_plain_xielu_both_sides_and_the_join():
    p, q = T(0.3), T(-0.2)
    ap, an = math.log1p(math.exp(0.3)), 0.5 + math.log1p(math.exp(-0.2))
    got = plain.xielu(T(2.0, -1.5, 0.0), p, q)
    assert got[0].item() == pytest.approx(ap * 4.0 + 1.0)
    assert got[1].item() == pytest.approx(an * (math.exp(-1.5) - 1 + 1.5) - 0.75)
    assert got[2].item() == 0.0
    # both sides leave zero with slope 1/2
    e = 1e-6
    lo, hi = plain.xielu(T(-e), p, q).item(), plain.xielu(T(e), p, q).item()
    assert lo == pytest.approx(-e / 2, rel=1e-4) and hi == pytest.approx(e / 2, rel=1e-4)


def test_plain_chunks_count_from_position_zero():
    vis = plain.chunk_mask(8, 3)
    assert vis[4].tolist() == [False, False, False, True, True, False, False, False]
    assert vis[5].tolist() == [False, False, False, True, True, True, False, False]
    assert vis[6].tolist() == [False] * 6 + [True, False]                              # a chunk's first position sees itself only
    assert plain.chunk_mask(4, None)[3].tolist() == [True] * 4


def test_plain_distance_penalty_is_zero_on_the_diagonal_and_grows_with_the_logarithm():
    b = plain.distance_penalty(5, T(2.0, 0.5), T(1.0, 3.0))
    assert b[0, 3, 3].item() == 0.0 and b[1, 4, 4].item() == 0.0
    assert b[0, 4, 1].item() == pytest.approx(2.0 * math.log(4.0))
    assert b[1, 4, 2].item() == pytest.approx(0.5 * math.log(7.0))


def test_plain_convolution_puts_the_last_tap_on_the_current_token():
    x = T([1.0], [2.0], [3.0])
    y = plain.causal_conv(x, T([10.0, 100.0, 1000.0]))
    assert y[:, 0].tolist() == [1000.0, 2000.0 + 100.0, 3000.0 + 200.0 + 10.0]


def test_plain_chunked_attention_two_tokens_by_hand():
    """One query head on one key/value head, sizes 2 and 2: the second token weighs both keys, with the penalty on the first;
    the values are divided by their root mean square before they are weighed."""
    g = torch.Generator().manual_seed(2)
    W = 3
    t = {n: torch.randn(s, generator=g, dtype=F64) for n, s in (("q", (2, W)), ("k", (2, W)), ("v", (2, W)), ("g", (2, W)),
                                                                    ("o", (W, 2)))}
    t["r1"], t["r2"] = T(0.7), T(1.9)
    mc = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.6, "mask": {"size": 4}}
    h = torch.randn(2, W, generator=g, dtype=F64)
    kv = plain.keys_values(h, t, "", mc, 1e-5)
    got = plain.chunked_attention(h, t, "", mc, 1e-5, kv)
    q, k, v = h @ t["q"].T, h @ t["k"].T, h @ t["v"].T
    vn = v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5)
    s0 = (q[1] * k[0]).sum() * 0.6 - 0.7 * math.log(1 + 1.9)
    s1 = (q[1] * k[1]).sum() * 0.6
    p0 = torch.exp(s0) / (torch.exp(s0) + torch.exp(s1))
    o = (p0 * vn[0] + (1 - p0) * vn[1]) * torch.sigmoid(h[1] @ t["g"].T)
    assert torch.allclose(got[1], o @ t["o"].T)
    assert torch.allclose(got[0], (vn[0] * torch.sigmoid(h[0] @ t["g"].T)) @ t["o"].T)
    # a chunk of one: every token sees itself alone
    alone = plain.chunked_attention(h, t, "", dict(mc, mask={"size": 1}), 1e-5, kv)
    assert torch.allclose(alone[1], (vn[1] * torch.sigmoid(h[1] @ t["g"].T)) @ t["o"].T)


def test_plain_delta_rule_first_steps_by_hand():
    """One head of size 1 x 1, two taps: S1 = beta1 v1 k1 (k1 = +-1 up to the floor), then the decay, the correction by what
    the state already answers for k2, and the read-out AFTER the write."""
    one = lambda x: torch.tensor([[x]], dtype=F64)
    t = {"q": one(1.5), "k": one(-2.0), "v": one(0.8), "b": one(0.4), "a1": one(1.0), "a2": one(0.6), "g1": one(1.0), "g2": one(0.0),
         "o": one(1.0), "q.conv": T([0.5, 2.0]), "k.conv": T([0.0, 1.0]), "v.conv": T([-1.0, 1.0]),
         "A_log": T(0.2), "dt_bias": T(-0.3), "norm": T(1.0)}
    mc = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 2}
    h = T([1.0], [0.5])
    y, (S, tail) = plain.channel_delta(h, t, "", mc, 0.0, return_state=True)
    silu = lambda z: z / (1 + math.exp(-z))
    unit = lambda z: z / math.sqrt(z * z + 1e-6)
    qc = [silu(2.0 * 1.5), silu(0.5 * 1.5 + 2.0 * 0.75)]
    kc = [silu(-2.0), silu(-1.0)]
    vc = [silu(0.8), silu(-0.8 + 0.4)]
    beta = [1 / (1 + math.exp(-0.4)), 1 / (1 + math.exp(-0.2))]
    dec = [math.exp(-math.exp(0.2) * math.log1p(math.exp(0.6 * x - 0.3))) for x in (1.0, 0.5)]
    s1 = beta[0] * vc[0] * unit(kc[0])
    sd = dec[1] * s1
    s2 = sd + unit(kc[1]) * beta[1] * (vc[1] - sd * unit(kc[1]))
    assert S.item() == pytest.approx(s2)
    assert tail.tolist() == [[0.5 * 1.5, 0.5 * -2.0, 0.5 * 0.8]]
    o2 = s2 * unit(qc[1])                                                            # dim^-1/2 = 1
    assert y[1].item() == pytest.approx(o2 / abs(o2) * 0.5)                           # unit rms of one number, gate sigmoid(0)
    # a portion continued from a state (matrix and convolution tail) equals the whole
    y1, st = plain.channel_delta(h[:1], t, "", mc, 0.0, return_state=True)
    y2 = plain.channel_delta(h[1:], t, "", mc, 0.0, state=st)
    assert torch.allclose(torch.cat([y1, y2]), y)


def test_plain_delta_rule_decay_acts_on_key_channels():
    """With beta -> 0 for the second token nothing is written, so S2 = diag(g) S1: rows (key channels) shrink, columns do
    not mix."""
    g = torch.Generator().manual_seed(5)
    D, V, W = 3, 2, 4
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    t = {"q": r(D, W), "k": r(D, W), "v": r(V, W), "b": r(1, W), "a1": r(2, W), "a2": r(D, 2), "g1": r(2, W), "g2": r(V, 2),
         "o": r(W, V), "q.conv": r(D, 1), "k.conv": r(D, 1), "v.conv": r(V, 1), "A_log": r(1), "dt_bias": r(D), "norm": r(V)}
    mc = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": V, "conv": 1}
    h = r(2, W)
    t["b"] = torch.linalg.lstsq(h, T([0.0], [-60.0])).solution.T                      # beta_1 = 1/2, beta_2 ~ 0
    _, (S1, _) = plain.channel_delta(h[:1], t, "", mc, 1e-6, return_state=True)
    _, (S2, _) = plain.channel_delta(h, t, "", mc, 1e-6, return_state=True)
    step = plain.softplus((h[1] @ t["a1"].T) @ t["a2"].T + t["dt_bias"])
    dec = torch.exp(-torch.exp(t["A_log"]) * step)
    assert torch.allclose(S2[0], dec[:, None] * S1[0], atol=1e-12)


def test_plain_latent_attention_one_token_and_the_shared_rotated_part():
    g = torch.Generator().manual_seed(7)
    H, D, R, V, rank, qr, W = 2, 3, 2, 2, 4, 3, 5
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    t = {"dq": r(qr, W), "dq.norm": r(qr), "uq": r(H * (D + R), qr), "dkv": r(rank + R, W), "dkv.norm": r(rank),
         "uk": r(H * D, rank), "uv": r(H * V, rank), "g": r(H * V, W), "o": r(W, H * V)}
    mc = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": rank, "q_rank": qr, "scale": 0.4, "rot": {"dims": R, "base": 50.0}}
    h = r(3, W)
    got = plain.latent_attention(h, t, "", mc, 1e-5)
    dkv = h @ t["dkv"].T
    c = plain.rms_norm(dkv[:, :rank], t["dkv.norm"], 1e-5)
    assert torch.allclose(got[0], ((c[0] @ t["uv"].T) * torch.sigmoid(h[0] @ t["g"].T)) @ t["o"].T)   # one key: weight 1
    # the score of head 1, query 2 on key 1, written out: unrotated part through the latent, rotated part shared
    cq = plain.rms_norm(h @ t["dq"].T, t["dq.norm"], 1e-5)
    q = (cq @ t["uq"].T).view(3, H, D + R)
    rot = lambda v, p: torch.stack([v[0] * math.cos(p) - v[1] * math.sin(p), v[1] * math.cos(p) + v[0] * math.sin(p)])
    scores = []
    for j in range(3):
        kn = (c[j] @ t["uk"].T).view(H, D)[1]
        scores.append(((q[2, 1, :D] * kn).sum() + (rot(q[2, 1, D:], 2.0) * rot(dkv[j, rank:], float(j))).sum()) * 0.4)
    p = torch.softmax(torch.stack(scores), 0)
    v = (c @ t["uv"].T).view(3, H, V)[:, 1]
    head1 = (p[:, None] * v).sum(0)
    o_all = plain.latent_attention(h, dict(t, o=torch.eye(H * V, dtype=F64)), "", mc, 1e-5)       # heads before Wo
    assert torch.allclose(o_all[2, V:], head1 * torch.sigmoid(h[2] @ t["g"].T)[V:])


def test_plain_token_side_and_cap():
    g = torch.Generator().manual_seed(9)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    t = {"gate": r(2, 3), "proj": r(3, 2), "norm": r(3)}
    x, e = r(1, 3), r(1, 2)
    z = x @ t["gate"].T
    gz = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    y = (gz * e) @ t["proj"].T
    assert torch.allclose(plain.token_side(x, e, t, "", 1e-5), y / torch.sqrt((y * y).mean() + 1e-5) * t["norm"])
    assert plain.tanh_cap(T(100.0, -0.01), 7.0).tolist() == pytest.approx([7.0, -0.01], rel=1e-5)


# ---- configuration and names --------------------------------------------------------------------------
def test_config_is_read_layer_by_layer():
    arch = architecture_of(CONFIGS["P"])
    assert arch.name == "Senadra"
    c = arch.load_config(CONFIGS["P"])
    assert [l.type for l in c.layers] == ["attention", "channel_delta", "latent_attention", "attention", "channel_delta"]
    assert c.layers[0].mixer.chunk == 24 and c.layers[3].mixer.kv_from == 0 and c.layers[3].mixer.chunk == 17
    assert c.layers[2].mlp is None and c.layers[2].mixer.rot_base == 30000.0 and c.layers[1].mixer.decay_rank == 6
    assert c.residual_mult == 0.45 and c.side_dim == 10 and c.logit_softcap == 8.0
    assert arch.load_config(arch.config_to_dict(c)) == c
    spec = arch.build_spec(c)
    assert [(o.layer, o.cache, o.writes_cache) for o in spec.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False),
                                                                         (4, 4, True)]
    assert spec.layers[3].mixer["owns_kv"] is False and spec.layers[2].mixer["position"]["style"] == "interleaved"
    r = arch.load_config(CONFIGS["R"])
    assert r.residual_mult == 1.0 and r.side_dim == 0 and r.logit_softcap is None and r.layers[4].mixer.chunk is None


def test_inner_sizes_of_the_low_rank_maps_come_from_the_tensors():
    arch = get_architecture("Senadra")
    raw = json.loads(json.dumps(CONFIGS["P"]))
    for lr in raw["layers"]:
        lr["mixer"].pop("decay_rank", None)
        lr["mixer"].pop("gate_rank", None)
    with pytest.raises(ConfigError, match="decay_rank"):
        arch.load_config(raw)
    shapes = {"l1.mix.a1": (6, 96), "l1.mix.g1": (9, 96), "l4.mix.a1": (5, 96), "l4.mix.g1": (3, 96)}
    assert arch.load_config(arch.with_tensor_sizes(raw, shapes)) == arch.load_config(CONFIGS["P"])


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="other"), "unknown type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="other"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "lacks 'kv_heads'"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "6 heads for 4"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "4 heads for 3"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "projects none"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=20), "heads differ"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c.update(logit_softcap=0.0), "logit_softcap"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_name_the_place(edit, text):
    raw = json.loads(json.dumps(CONFIGS["P"]))
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        get_architecture("Senadra").load_config(raw)


def test_tensor_names_and_cache_needs(tmp_path):
    arch = get_architecture("Senadra")
    names = declare_tensors(arch, arch.build_spec(arch.load_config(CONFIGS["P"])))
    for n in ("embed", "side.embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.r1",
              "l0.mix.r2", "l0.mix.g", "l0.mix.o", "l0.mlp.up", "l0.mlp.down", "l0.mlp.act", "l0.side.gate", "l0.side.proj",
              "l0.side.norm", "l1.mix.q.conv", "l1.mix.k.conv", "l1.mix.v.conv", "l1.mix.b", "l1.mix.A_log", "l1.mix.a1", "l1.mix.a2",
              "l1.mix.dt_bias", "l1.mix.g1", "l1.mix.g2", "l1.mix.norm", "l2.mix.dq", "l2.mix.dq.norm", "l2.mix.uq", "l2.mix.dkv",
              "l2.mix.dkv.norm", "l2.mix.uk", "l2.mix.uv", "l2.mix.g", "l3.mix.q", "l3.mix.r1", "l4.side.norm"):
        assert n in names, n
    for n in ("l3.mix.k", "l3.mix.v", "l2.mlp.up", "l2.norm2", "l4.mlp.act", "l0.mlp.gate"):
        assert n not in names, n
    assert names["side.embed"].shape == (211, 50) and names["l0.mix.v"].shape == (48, 96) and names["l0.mix.g"].shape == (144, 96)
    assert names["l1.mix.a2"].shape == (48, 6) and names["l1.mix.q.conv"].shape == (24, 4) and names["l1.mix.norm"].shape == (20,)
    assert names["l2.mix.dkv"].shape == (48, 96) and names["l2.mix.uq"].shape == (72, 28) and names["l0.mlp.act"].shape == (2,)
    d = write_case(tmp_path, "P", store_dtype=torch.float32)
    with ops.use_kernels(FakeKernels()):
        needs = Model.from_folder(d, "float32", "cpu").cache_needs()
    assert sorted(needs) == [0, 1, 2, 4]                                               # the reader of layer 0's pages has none
    assert needs[0] == KVNeed(2, 16, None, 24) and needs[2] == RowNeed(48)
    assert isinstance(needs[1], StateNeed) and needs[1].dtype == torch.float32
    assert needs[1].shape == (4 * 20 * 12 + 3 * (2 * 2 * 12 + 4 * 20),) and needs[4].shape == (2 * 8 * 40 + 1 * (2 * 2 * 40 + 2 * 8),)


# ---- the host side under every way of cutting the work -------------------------------------------------
@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("senadra")
    out = {}
    for name in CONFIGS:
        d = write_case(root, name, store_dtype=torch.float32)
        with ops.use_kernels(FakeKernels()):
            out[name] = (d, Model.from_folder(d, "float32", "cpu"))
    return out


LENGTHS = {"P": [1, 9, 40, 75], "Q": [3, 35, 70, 20, 2], "R": [2, 90, 33], "S": [45, 5, 20], "T": [41, 3, 30]}


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


def test_plain_forward_gives_the_stream_after_every_layer(cases):
    """The GPU tests compare the engine's stream layer by layer with this; a layer that reads another's keys and values moves
    the stream like any other."""
    d, _ = cases["P"]
    cfg, w = plain.load_folder(d)
    toks = random_tokens(211, 30, 77)
    logits, layers = plain.forward(cfg, w, toks, return_layers=True)
    assert layers.shape == (5, 30, 96) and logits.shape == (30, 211)
    assert (layers[3] - layers[2]).abs().max() > 1e-3
    assert logits.abs().max() < 8.0                                                    # the cap


def test_a_slot_that_is_used_again_starts_from_zero(cases):
    """Two state slots, five requests one after another and side by side: a request that inherits a slot must see neither
    the matrix nor the convolution tail that the one before left in it."""
    d, model = cases["P"]
    reqs = {f"r{i}": random_tokens(211, n, 90 + i) for i, n in enumerate([30, 12, 25, 7, 18])}
    want = plain_logits(d, reqs)
    steps = trace_mixed(reqs, 128, seed=1, max_live=2)
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 2, native=False)
        got = replay_and_collect(rp, steps)
    bad = first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong logits at {bad}"


def test_portions_of_two_tokens_and_single_tokens_across_chunk_edges(cases):
    """Chunks of 24 and 17 positions under pages of 16: portions of two tokens and single tokens walk over every edge."""
    d, model = cases["P"]
    toks = random_tokens(211, 60, 8)
    want = plain_logits(d, {"a": toks})["a"]
    for size in (2, 1, 5):
        steps = [{"step": i, "entries": [{"id": "a", "tokens": toks[p:p + size], "want": list(range(len(toks[p:p + size])))}],
                  "end": []} for i, p in enumerate(range(0, 60, size))]
        with ops.use_kernels(FakeKernels()):
            rp = TraceReplayer(model, 64, 16, 4, native=False)
            got = torch.cat([rp.run_step(s).clone() for s in steps]).double()
        assert (got - want).abs().max() < 2e-4, size


def test_greedy_generation_through_the_scheduler(cases):
    d, model = cases["Q"]
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
    """``iian random-weights`` from a Senadra config.json, then the folder through the loader (names, shapes, the plug-in); the
    inner sizes of the low-rank maps are then read back from the tensors' shapes."""
    from iian_b200.cli.main import main as cli_main
    from iian_b200.config.registry import load_model_config
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["R"]))
    out = tmp_path / "model"
    assert cli_main(["random-weights", str(cfg_path), str(out), "--seed", "3"]) == 0
    # take the ranks out of the written config.json: the loader finds them in the weight file
    written = json.loads((out / "config.json").read_text())
    for lr in written["layers"]:
        lr["mixer"].pop("decay_rank", None)
        lr["mixer"].pop("gate_rank", None)
    (out / "config.json").write_text(json.dumps(written))
    arch, cfg = load_model_config(str(out))
    assert arch.name == "Senadra" and cfg == arch.load_config(CONFIGS["R"])
    with ops.use_kernels(FakeKernels()):
        model = Model.from_folder(str(out), "float32", "cpu")
        rp = TraceReplayer(model, 64, 16, 2, native=False)
        logits = rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]})
    want = plain.forward(*plain.load_folder(str(out)), [1, 2, 3])[-1]
    assert (logits[0].double() - want).abs().max() < 2e-4
