"""The kernels of the Galodra design alone, each beside the like kernel of the Qwen3 path at equal size.

    python -m iian_b200.cli.design_kernels            (or ``bench.py --design galodra --kernels``)

A kernel is timed as a replayed CUDA graph of a few launches on different copies of its operands (which together exceed
the L2 wherever memory is the bound), after one eager run, with a 256 MB buffer written before every replay; the median
of several replays counts (a graph of ONE short launch cannot read below some 16 us, hence several).  Achieved bytes or
flops are the algorithmic ones (what the operation has to read and write, or multiply) over that time, set against the measured copy
bandwidth and bfloat16 product peak.

Pairs (width 2048, 16 heads; latent rank 512 + 64 rotated; Qwen3 side: 16 heads of 128 on 8 KV heads):
  decode attention   8 (and 64) sequences of 4,096 cached tokens, one new token each   bytes of cache read
  prefill attention  one sequence of 2,048 tokens                                 flops of scores and values
  expert products    2,048 tokens x 6 of 64 experts (1,408 wide)  vs  the dense gate/up and down products of 8,448
  sum + norm         2,048 rows: gated sum with LayerNorm  vs  residual add with RMSNorm
  per-head products  the query into latent space and the values out of it (no like kernel on the Qwen3 path)
"""
from __future__ import annotations

import json
import statistics
import sys
from types import SimpleNamespace


def _timed(fns, iters: int = 7) -> float:
    """Median milliseconds of one call: the calls of ``fns`` (the same kernel on different copies of its operands, which
    together exceed the L2) run once eagerly, are then captured into one CUDA graph, and the graph is replayed ``iters``
    times, each time after a 256 MB buffer was written; a replay's device time over the number of calls counts.  Timing
    a graph keeps the host's launch cost out of kernels of a few microseconds."""
    import torch
    if callable(fns):
        fns = [fns]
    flush = _timed.flush
    if flush is None:
        flush = _timed.flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / len(fns))
    return statistics.median(times)


_timed.flush = None


def _meta(ctx_lens, q_lens, page: int, dev):
    import torch
    n_blocks = [-(-c // page) for c in ctx_lens]
    bt = torch.full((len(ctx_lens), max(n_blocks)), -1, dtype=torch.int32)
    nxt, positions, seq, cu = 0, [], [], [0]
    for s, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        bt[s, : n_blocks[s]] = torch.arange(nxt, nxt + n_blocks[s], dtype=torch.int32)
        nxt += n_blocks[s]
        positions += list(range(c - ql, c))
        seq += [s] * ql
        cu.append(cu[-1] + ql)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    return SimpleNamespace(positions=t(positions), seq_of_token=t(seq), cu_q=t(cu), ctx_len=t(ctx_lens), block_table=bt.to(dev),
                           slots=None, num_seqs=len(ctx_lens), num_tokens=len(positions), max_q_len=max(q_lens), max_ctx=max(ctx_lens),
                           decode_only=max(q_lens) == 1, h_q_len=list(q_lens), h_ctx_len=list(ctx_lens)), nxt


def run(peaks: dict, width: int = 2048, heads: int = 16) -> dict:
    import torch
    from .. import ops
    from ..config.spec import PartSpec
    from ..engine.runner import StepContext, Workspace
    from ..parts.experts import RoutedExperts
    k = ops.kernels()
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    rank, rot, dim, vdim, page, window = 512, 64, 128, 128, 16, 4096
    lw = rank + rot
    out = {}
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]

    def mem_row(name, ms, nbytes):
        out[name] = {"ms": ms, "gb_s": nbytes / ms / 1e6, "of_hbm_peak": nbytes / ms / 1e6 / hbm}

    def flop_row(name, ms, flops):
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "of_bf16_peak": flops / ms / 1e9 / tfl}

    # ---- decode attention: a short step (bound by its fixed costs: two launches, the first tile, the merge) and a long one ----
    sink = torch.zeros(heads, device=dev)
    nkv, hd = 8, 128
    for B, ctx in ((8, 4096), (64, 4096)):
        tag = "" if B == 8 else f"_{B}x{ctx}"
        meta, pages = _meta([ctx] * B, [1] * B, page, dev)
        n_copies = 5 if B == 8 else 2
        copies = [torch.randn(pages, page, lw, device=dev).to(bf) * 0.3 for _ in range(n_copies)]
        q = torch.randn(B, heads, lw, device=dev).to(bf) * 0.1
        o = torch.empty(B, heads, rank, device=dev, dtype=bf)
        ms = _timed([(lambda r=r: k.latent_attention_mma(q, r, o, sink, meta, num_heads=heads, rank=rank, scale=0.07, window=window))
                     for r in copies])
        mem_row("decode_attention_latent" + tag, ms, B * ctx * lw * 2)
        del copies
        n_copies = 3 if B == 8 else 2
        copies = [(torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3, torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3)
                  for _ in range(n_copies)]
        q2 = torch.randn(B, heads, hd, device=dev).to(bf) * 0.1
        o2 = torch.empty(B, heads * hd, device=dev, dtype=bf)
        ms = _timed([(lambda c=c: k.paged_attention(q2, c[0], c[1], o2, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                                    window=window)) for c in copies])
        mem_row("decode_attention_qwen3" + tag, ms, B * ctx * 2 * nkv * hd * 2)
        del copies
    torch.cuda.empty_cache()

    # ---- prefill attention -------------------------------------------------------------------------------------------
    T = 2048
    meta, pages = _meta([T], [T], page, dev)
    rows = torch.randn(pages, page, lw, device=dev).to(bf) * 0.3
    q = torch.randn(T, heads, lw, device=dev).to(bf) * 0.1
    o = torch.empty(T, heads, rank, device=dev, dtype=bf)
    pairs = T * (T + 1) / 2
    ms = _timed(lambda: k.latent_attention_mma(q, rows, o, sink, meta, num_heads=heads, rank=rank, scale=0.07, window=window))
    flop_row("prefill_attention_latent", ms, 2.0 * heads * (lw + rank) * pairs)
    kc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    vc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    q2 = torch.randn(T, heads, hd, device=dev).to(bf) * 0.1
    o2 = torch.empty(T, heads * hd, device=dev, dtype=bf)
    ms = _timed([lambda: k.paged_attention(q2, kc, vc, o2, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088, window=window)] * 4)
    flop_row("prefill_attention_qwen3", ms, 4.0 * heads * hd * pairs)

    # ---- expert products beside the dense products of the same active size -------------------------------------------
    E, top, ff = 64, 6, 1408
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "num_experts": E, "top": top, "intermediate_size": ff}),
                         bf, dev)
    tensors = {"router": torch.randn(E, width, device=dev).to(bf) * 0.05}
    for e in range(E):
        tensors[f"e{e}.gate"] = torch.randn(ff, width, device=dev).to(bf) * 0.02
        tensors[f"e{e}.up"] = torch.randn(ff, width, device=dev).to(bf) * 0.02
        tensors[f"e{e}.down"] = torch.randn(width, ff, device=dev).to(bf) * 0.02
    part.bind(tensors)
    del tensors
    for n in (2048, 8):
        h = torch.randn(n, width, device=dev).to(bf)
        ctx_ = StepContext(Workspace(dev))
        part.forward(h, ctx_)                   # sizes the buffers and leaves a plan
        m = n * top
        offsets, tiles = ctx_.buf("expert_offsets", (E + 1,), torch.int32), ctx_.buf("expert_tiles", (1 + 2 * k.moe_max_tiles(m, E, 128),), torch.int32)
        xs, act, ys = ctx_.buf("expert_in", (m, width), bf), ctx_.buf("expert_act", (m, ff), bf), ctx_.buf("expert_out", (m, width), bf)
        ms1 = _timed(lambda: k.moe_grouped_gemm_tc(xs, part.w_gate_up, act, offsets, tiles, gated=True))
        ms2 = _timed(lambda: k.moe_grouped_gemm_tc(act, part.w_down, ys, offsets, tiles, gated=False))
        ms_all = _timed(lambda: part.forward(h, ctx_))
        if n >= 128:
            flop_row(f"expert_gate_up_{n}", ms1, 2.0 * m * 2 * ff * width)
            flop_row(f"expert_down_{n}", ms2, 2.0 * m * ff * width)
            flop_row(f"expert_feed_forward_{n}", ms_all, 2.0 * m * 3 * ff * width)
        else:
            reached = len(set(ctx_.buf("expert_ids", (n, top), torch.int32).flatten().tolist()))
            mem_row(f"expert_gate_up_{n}", ms1, reached * 2 * ff * width * 2)
            mem_row(f"expert_down_{n}", ms2, reached * ff * width * 2)
            mem_row(f"expert_feed_forward_{n}", ms_all, reached * 3 * ff * width * 2)
        inter = top * ff
        wgu = torch.randn(2 * inter, width, device=dev).to(bf) * 0.02
        wd = torch.randn(width, inter, device=dev).to(bf) * 0.02
        a2, y2 = torch.empty(n, inter, device=dev, dtype=bf), torch.empty(n, width, device=dev, dtype=bf)
        fused = k.can_fuse_swiglu(h, wgu, 8)
        gu = torch.empty(n, 2 * inter, device=dev, dtype=bf)

        def dense_gate_up():
            if fused:
                k.linear_swiglu(h, wgu, a2)
            else:
                k.linear(h, wgu, gu)
                k.swiglu(gu, a2, 8)
        # at 8 tokens the weights are the traffic: three copies (207 MB) so that none waits in the L2
        wgus = [wgu] + [wgu.clone() for _ in range(2 if n < 128 else 0)]
        wds = [wd] + [wd.clone() for _ in range(5 if n < 128 else 0)]

        def dense_gate_up_on(wm):
            def run_():
                if fused:
                    k.linear_swiglu(h, wm, a2)
                else:
                    k.linear(h, wm, gu)
                    k.swiglu(gu, a2, 8)
            return run_
        ms1 = _timed([dense_gate_up_on(wm) for wm in wgus] * (1 if n < 128 else 3))
        ms2 = _timed([(lambda wm=wm: k.linear(a2, wm, y2)) for wm in wds] * (1 if n < 128 else 3))
        del wgus, wds
        if n >= 128:
            flop_row(f"dense_gate_up_{n}", ms1, 2.0 * n * 2 * inter * width)
            flop_row(f"dense_down_{n}", ms2, 2.0 * n * inter * width)
        else:
            mem_row(f"dense_gate_up_{n}", ms1, 2 * inter * width * 2)
            mem_row(f"dense_down_{n}", ms2, inter * width * 2)
        del wgu, wd

    # ---- sum + norm ----------------------------------------------------------------------------------------------------
    n = 2048
    x = torch.randn(n, width, device=dev)
    sub = torch.randn(n, width, device=dev).to(bf)
    gate = torch.randn(n, width, device=dev).to(bf)
    gb, w, b = torch.zeros(width, device=dev), torch.ones(width, device=dev), torch.zeros(width, device=dev)
    o32, o16 = torch.empty(n, width, device=dev), torch.empty(n, width, device=dev, dtype=bf)
    sets = [(x.clone(), sub.clone(), gate.clone(), torch.empty_like(o32), torch.empty_like(o16)) for _ in range(8)]
    ms = _timed([(lambda t=t: k.gated_add_layer_norm(t[0], t[1], t[2], gb, w, b, 2.0, 1e-6, t[3], t[4])) for t in sets])
    mem_row("gated_sum_layer_norm", ms, n * width * (4 + 2 + 2 + 4 + 2))
    ms = _timed([(lambda t=t: k.add_rms_norm(t[0], t[1], w, 1e-6, t[4])) for t in sets])         # 8 x 32 MB: twice the L2
    mem_row("add_rms_norm_qwen3", ms, n * width * (4 + 2 + 4 + 2))
    del sets
    coef = torch.ones(5, device=dev)
    sets = [[torch.randn(n, width, device=dev) for _ in range(5)] for _ in range(3)]
    ms = _timed([(lambda t=t: k.depth_mix(t, coef, None, False, o32, o16)) for t in sets])
    mem_row("depth_mix_5_terms", ms, n * width * (5 * 4 + 4 + 2))
    del sets

    # ---- per-head products ---------------------------------------------------------------------------------------------
    for n in (2048, 8):
        qd = torch.randn(n, heads * (dim + rot), device=dev).to(bf)
        uk = torch.randn(heads * dim, rank, device=dev).to(bf) * 0.05
        q_cat = torch.empty(n, heads * lw, device=dev, dtype=bf)
        uks = [uk.clone() for _ in range(70 if n <= 8 else 1)] * (1 if n <= 8 else 8)        # many rows: flop-bound, operands may wait in the L2
        ms = _timed([(lambda u=u: k.head_linear(qd, 0, dim + rot, u, dim * rank, rank, 1, q_cat, 0, lw, num_heads=heads, n_in=dim, n_out=rank))
                     for u in uks])
        (flop_row if n >= 128 else mem_row)(f"query_into_latent_{n}", ms, 2.0 * n * heads * dim * rank if n >= 128 else heads * dim * rank * 2)
        lat = torch.randn(n, heads * rank, device=dev).to(bf)
        uv = torch.randn(heads * vdim, rank, device=dev).to(bf) * 0.05
        hv = torch.empty(n, heads * vdim, device=dev, dtype=bf)
        uvs = [uv.clone() for _ in range(70 if n <= 8 else 1)] * (1 if n <= 8 else 8)
        ms = _timed([(lambda u=u: k.head_linear(lat, 0, rank, u, vdim * rank, 1, rank, hv, 0, vdim, num_heads=heads, n_in=rank, n_out=vdim))
                     for u in uvs])
        (flop_row if n >= 128 else mem_row)(f"values_out_of_latent_{n}", ms, 2.0 * n * heads * vdim * rank if n >= 128 else heads * vdim * rank * 2)
    k.check_device_status()
    return out


def run_lekilix(peaks: dict, width: int = 2048, heads: int = 16) -> dict:
    """The kernels of the Lekilix design alone, each beside the like kernel of the Qwen3 path at equal size (16 heads of 128 on
    8 KV heads, window 4,096; memories of 8 heads, 128 deep and 256 wide):
      decode attention    8 (and 64) sequences of 4,096 cached tokens: with the sink  vs  without      bytes of cache read
      prefill attention   one sequence of 2,048 tokens                                                  flops of scores and values
      norm + rotation     2,048 tokens: norm over the whole projection, values = keys  vs  per-head norm, separate values
      sum + norm          2,048 rows: two sub-layer outputs in the sum  vs  one
      expert products     2,048 tokens x 6 of 64 experts by table (1,408 wide)  vs  the dense products of 8,448
      memory scan         8 / 64 sequences of one token (bytes of state) and one sequence of 2,048 tokens (no like kernel)
    """
    import torch
    from .. import ops
    from ..config.spec import PartSpec
    from ..engine.runner import StepContext, Workspace
    from ..parts.experts import RoutedExperts
    from ..parts.matrix_memory import state_block_floats, state_columns
    k = ops.kernels()
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    nkv, hd, page, window = 8, 128, 16, 4096
    out = {}
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]

    def mem_row(name, ms, nbytes):
        out[name] = {"ms": ms, "gb_s": nbytes / ms / 1e6, "of_hbm_peak": nbytes / ms / 1e6 / hbm}

    def flop_row(name, ms, flops):
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "of_bf16_peak": flops / ms / 1e9 / tfl}

    sink = torch.randn(heads, device=dev)
    # ---- decode attention ------------------------------------------------------------------------------------------------
    for B, ctx in ((8, 4096), (64, 4096)):
        meta, pages = _meta([ctx] * B, [1] * B, page, dev)
        copies = [(torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3, torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3)
                  for _ in range(3 if B == 8 else 2)]
        q = torch.randn(B, heads, hd, device=dev).to(bf) * 0.1
        o = torch.empty(B, heads * hd, device=dev, dtype=bf)
        nbytes = B * ctx * 2 * nkv * hd * 2
        ms = _timed([(lambda c=c: k.sink_attention(q, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                                   window=window, sink=sink)) for c in copies])
        mem_row(f"decode_attention_sink_{B}x{ctx}", ms, nbytes)
        ms = _timed([(lambda c=c: k.paged_attention(q, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                                    window=window)) for c in copies])
        mem_row(f"decode_attention_qwen3_{B}x{ctx}", ms, nbytes)
        del copies
    torch.cuda.empty_cache()
    # ---- prefill attention -----------------------------------------------------------------------------------------------
    T = 2048
    meta, pages = _meta([T], [T], page, dev)
    kc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    vc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    q = torch.randn(T, heads, hd, device=dev).to(bf) * 0.1
    o = torch.empty(T, heads * hd, device=dev, dtype=bf)
    pairs = T * (T + 1) / 2
    ms = _timed([lambda: k.sink_attention(q, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088, window=window,
                                          sink=sink)] * 4)
    flop_row("prefill_attention_sink", ms, 4.0 * heads * hd * pairs)
    ms = _timed([lambda: k.paged_attention(q, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088, window=window)] * 4)
    flop_row("prefill_attention_qwen3", ms, 4.0 * heads * hd * pairs)
    # ---- norm, rotation, cache write ---------------------------------------------------------------------------------------
    slots = torch.arange(T, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    wide = (2 * heads + nkv) * hd
    sets = [(torch.randn(T, wide, device=dev).to(bf), torch.empty(T, heads, hd, device=dev, dtype=bf), torch.zeros_like(kc), torch.zeros_like(vc))
            for _ in range(4)]
    qw, kw = torch.ones(heads * hd, device=dev), torch.ones(nkv * hd, device=dev)
    inv64 = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -torch.arange(32, dtype=torch.float64) / 32).to(dev)
    ms = _timed([(lambda t=t: k.projection_norm_rope_store(t[0], 0, heads * hd, t[1], t[2], t[3], num_heads=heads, num_kv_heads=nkv,
                                                           head_dim=hd, q_weight=qw, k_weight=kw, eps=1e-6, inv_freq=inv64, rot_dim=64,
                                                           rope_style=1, positions=pos, slots=slots)) for t in sets])
    mem_row("projection_norm_rope_store", ms, T * (heads + nkv) * hd * 2 + T * (heads + 2 * nkv) * hd * 2)
    sets2 = [(torch.randn(T, (heads + 2 * nkv) * hd, device=dev).to(bf), t[1], t[2], t[3]) for t in sets]
    qw2, kw2 = torch.ones(hd, device=dev), torch.ones(hd, device=dev)
    inv_full = torch.pow(torch.tensor(500000.0), -torch.arange(hd // 2, dtype=torch.float32) / (hd // 2)).to(dev)
    ms = _timed([(lambda t=t: k.qk_norm_rope_store(t[0], t[1], t[2], t[3], num_heads=heads, num_kv_heads=nkv, head_dim=hd, q_weight=qw2,
                                                   k_weight=kw2, eps=1e-6, inv_freq=inv_full, rot_dim=hd, rope_style=0, positions=pos,
                                                   slots=slots, write_kv=True)) for t in sets2])
    mem_row("qk_norm_rope_store_qwen3", ms, 2 * T * (heads + 2 * nkv) * hd * 2)
    del sets, sets2, kc, vc
    # ---- sum + norm ------------------------------------------------------------------------------------------------------------
    n = 2048
    w = torch.ones(width, device=dev)
    sets = [(torch.randn(n, width, device=dev), torch.randn(n, width, device=dev).to(bf), torch.randn(n, width, device=dev).to(bf),
             torch.empty(n, width, device=dev, dtype=bf)) for _ in range(8)]
    ms = _timed([(lambda t=t: k.add2_rms_norm(t[0], t[1], t[2], w, 1e-6, t[3])) for t in sets])
    mem_row("add2_rms_norm", ms, n * width * (4 + 2 + 2 + 4 + 2))
    ms = _timed([(lambda t=t: k.add_rms_norm(t[0], t[1], w, 1e-6, t[3])) for t in sets])
    mem_row("add_rms_norm_qwen3", ms, n * width * (4 + 2 + 4 + 2))
    del sets
    # ---- expert products beside the dense products of the same active size ---------------------------------------------------------
    E, top, ff, vocab = 64, 6, 1408, 32768
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "num_experts": E, "top": top, "intermediate_size": ff,
                                                     "activation": "clamped_swish", "limit": 7.0, "score": "table", "vocab_size": vocab,
                                                     "weight_on": "output"}), bf, dev)
    tensors = {"table": torch.stack([torch.randperm(E)[:top] for _ in range(vocab)]).to(torch.int32).to(dev)}
    for e in range(E):
        tensors[f"e{e}.gate"] = torch.randn(ff, width, device=dev).to(bf) * 0.02
        tensors[f"e{e}.up"] = torch.randn(ff, width, device=dev).to(bf) * 0.02
        tensors[f"e{e}.down"] = torch.randn(width, ff, device=dev).to(bf) * 0.02
    part.bind(tensors)
    del tensors
    for n in (2048, 8):
        h = torch.randn(n, width, device=dev).to(bf)
        ctx_ = StepContext(Workspace(dev))
        ctx_.tokens = torch.randint(0, vocab, (n,), device=dev).to(torch.int32)
        part.forward(h, ctx_)
        m = n * top
        ms_all = _timed(lambda: part.forward(h, ctx_))
        inter = top * ff
        wgu = torch.randn(2 * inter, width, device=dev).to(bf) * 0.02
        wd = torch.randn(width, inter, device=dev).to(bf) * 0.02
        a2, y2 = torch.empty(n, inter, device=dev, dtype=bf), torch.empty(n, width, device=dev, dtype=bf)
        fused = k.can_fuse_swiglu(h, wgu, 8)
        gu = torch.empty(n, 2 * inter, device=dev, dtype=bf)
        wgus = [wgu] + [wgu.clone() for _ in range(2 if n < 128 else 0)]
        wds = [wd] + [wd.clone() for _ in range(2 if n < 128 else 0)]

        def dense_on(wa, wb):
            def run_():
                if fused:
                    k.linear_swiglu(h, wa, a2)
                else:
                    k.linear(h, wa, gu)
                    k.swiglu(gu, a2, 8)
                k.linear(a2, wb, y2)
            return run_
        ms_dense = _timed([dense_on(a, b) for a, b in zip(wgus, wds)] * (1 if n < 128 else 3))
        if n >= 128:
            flop_row(f"expert_feed_forward_{n}", ms_all, 2.0 * m * 3 * ff * width)
            flop_row(f"dense_feed_forward_{n}", ms_dense, 2.0 * n * 3 * inter * width)
        else:
            reached = len(set(ctx_.buf("expert_ids", (n, top), torch.int32).flatten().tolist()))
            mem_row(f"expert_feed_forward_{n}", ms_all, reached * 3 * ff * width * 2)
            mem_row(f"dense_feed_forward_{n}", ms_dense, 3 * inter * width * 2)
        del wgus, wds, wgu, wd
    del part
    torch.cuda.empty_cache()
    # ---- the matrix-memory scan and what follows it ----------------------------------------------------------------------------------
    H, d, dv, cap = heads // 2, 128, 256, 15.0
    cb = state_columns(d, dv)
    wide = 2 * H * d + 2 * H * dv
    bias = torch.zeros(2 * H, device=dev)
    for B, L in ((8, 1), (64, 1), (1, 2048)):
        n = B * L
        sets = [(torch.randn(n, wide, device=dev).to(bf) * 0.5, torch.randn(n, 2 * H, device=dev),
                 torch.zeros(B, H, dv // cb, state_block_floats(d, cb), device=dev), torch.empty(n, H * dv, device=dev))
                for _ in range(4 if L == 1 else 1)]
        cu = torch.arange(0, n + 1, L, dtype=torch.int32, device=dev)
        sl = torch.arange(B, dtype=torch.int32, device=dev)
        ms = _timed([(lambda t=t: k.matrix_memory_scan(t[0], 0, H * d, 2 * H * d, t[1], bias, t[2], cu, sl, t[3], num_heads=H, dim=d,
                                                       v_dim=dv, columns=cb, cap=cap, q_scale=d ** -0.5, max_q_len=L)) for t in sets])
        if L == 1:
            mem_row(f"memory_scan_decode_{B}", ms, B * 2 * H * (d * dv + d) * 4)
        else:
            flop_row(f"memory_scan_prefill_{L}", ms, 4.0 * L * H * d * (dv + 1))
        if L > 1:
            gate = sets[0][0][:, 2 * H * d + H * dv:]
            wn = torch.ones(H * dv, device=dev)
            o16 = torch.empty(n, H * dv, device=dev, dtype=bf)
            ms = _timed([lambda: k.head_norm_gate(sets[0][3], wn, gate, o16, num_heads=H, eps=1e-6)] * 4)
            mem_row("head_norm_gate", ms, n * H * dv * (4 + 2 + 2))
        del sets
    k.check_device_status()
    return out


def run_nogelorn(peaks: dict, width: int = 2048, heads: int = 16) -> dict:
    """The kernels of the Nogelorn design alone, each beside its like kernel of the Lekilix path at equal size (16 heads of 128
    on 8 KV heads, window 4,096 with 128 kept first keys; recurrences of 8 heads, 128 deep and 256 wide):
      decode attention    8 (and 64) sequences of 6,144 cached tokens: window, kept keys, sink, head gate  vs  window and sink
      prefill attention   one sequence of 2,048 tokens, and of 8,192 (the window passes, the kept keys stay)   flops of scores and values
      rotation + cache    2,048 tokens: rotation, unit norm, cache write  vs  norm over the projection, rotation, cache write
      sum + norm          2,048 rows: a normalised addend in the next norm's sum  vs  two plain addends
      expert products     2,048 (and 8) tokens x 5 of 64 experts by softmax over the chosen logits + a shared one  vs  6 by table
      decayed scan        8 / 64 sequences of one token (bytes of state) and one sequence of 2,048 tokens, constant decay per
                          head and decay per channel  vs  the matrix-memory scan
    """
    import torch
    from .. import ops
    from ..config.spec import PartSpec
    from ..engine.runner import StepContext, Workspace
    from ..parts.experts import RoutedExperts
    from ..parts.matrix_memory import state_block_floats, state_columns
    k = ops.kernels()
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    nkv, hd, page, window, keep = 8, 128, 16, 4096, 128
    out = {}
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]

    def mem_row(name, ms, nbytes):
        out[name] = {"ms": ms, "gb_s": nbytes / ms / 1e6, "of_hbm_peak": nbytes / ms / 1e6 / hbm}

    def flop_row(name, ms, flops):
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "of_bf16_peak": flops / ms / 1e9 / tfl}

    sink = torch.randn(heads, device=dev)
    # ---- decode attention: contexts longer than the window, so that the kept keys are a stretch of their own ---------------
    for B, ctx in ((8, 6144), (64, 6144)):
        meta, pages = _meta([ctx] * B, [1] * B, page, dev)
        copies = [(torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3, torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3)
                  for _ in range(2)]
        q = torch.randn(B, heads * hd, device=dev).to(bf) * 0.1
        gate = torch.randn(B, heads, device=dev).to(bf)
        o = torch.empty(B, heads * hd, device=dev, dtype=bf)
        ms = _timed([(lambda c=c: k.window_attention(q, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, k_dim=hd, v_dim=hd,
                                                     scale=0.088, window=window, keep_first=keep, sink=sink, gate=gate, gate_per_head=True))
                     for c in copies])
        mem_row(f"decode_attention_kept_{B}x{ctx}", ms, B * (window + keep) * 2 * nkv * hd * 2)
        q3 = q.view(B, heads, hd)
        ms = _timed([(lambda c=c: k.sink_attention(q3, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                                   window=window, sink=sink)) for c in copies])
        mem_row(f"decode_attention_lekilix_{B}x{ctx}", ms, B * window * 2 * nkv * hd * 2)
        del copies
    torch.cuda.empty_cache()
    # ---- prefill attention -----------------------------------------------------------------------------------------------
    for T in (2048, 8192):
        meta, pages = _meta([T], [T], page, dev)
        kc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
        vc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
        q = torch.randn(T, heads * hd, device=dev).to(bf) * 0.1
        gate = torch.randn(T, heads, device=dev).to(bf)
        o = torch.empty(T, heads * hd, device=dev, dtype=bf)
        pairs = T * (T + 1) / 2 if T <= window else window * (window + 1) / 2 + (T - window) * window
        kept_pairs = pairs + (max(0, T - window - keep) * keep if T > window else 0)
        ms = _timed([lambda: k.window_attention(q, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, k_dim=hd, v_dim=hd, scale=0.088,
                                                window=window, keep_first=keep, sink=sink, gate=gate, gate_per_head=True)] * 3)
        flop_row(f"prefill_attention_kept_{T}", ms, 4.0 * heads * hd * kept_pairs)
        q3 = q.view(T, heads, hd)
        ms = _timed([lambda: k.sink_attention(q3, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                              window=window, sink=sink)] * 3)
        flop_row(f"prefill_attention_lekilix_{T}", ms, 4.0 * heads * hd * pairs)
        del kc, vc
    torch.cuda.empty_cache()
    # ---- rotation, unit norm, cache write ------------------------------------------------------------------------------------
    T = 2048
    meta, pages = _meta([T], [T], page, dev)
    slots = torch.arange(T, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    wide = (heads + 2 * nkv) * hd
    sets = [(torch.randn(T, wide, device=dev).to(bf), torch.empty(T, heads, hd, device=dev, dtype=bf),
             torch.zeros(pages, nkv, page, hd, device=dev, dtype=bf), torch.zeros(pages, nkv, page, hd, device=dev, dtype=bf)) for _ in range(4)]
    inv64 = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -torch.arange(hd // 2, dtype=torch.float64) / (hd // 2)).to(dev)
    table = torch.empty(T, hd // 2, 2, device=dev)
    k.rotary_table_scaled(inv64, pos, hd // 2, 1.0, table)
    ms = _timed([(lambda t=t: k.rotate_unit_store(t[0], 0, heads * hd, (heads + nkv) * hd, t[1], t[2], t[3], table, slots, num_heads=heads,
                                                  num_kv_heads=nkv, k_dim=hd, v_dim=hd, rot_dim=hd, eps=1e-6, unit_norm=True)) for t in sets])
    mem_row("rotate_unit_store", ms, 2 * T * (heads + 2 * nkv) * hd * 2)
    ms = _timed([lambda: k.rotary_table_scaled(inv64, pos, hd // 2, 1.0, table)] * 4)
    mem_row("rotary_table_float64_angles", ms, T * hd // 2 * 8)
    sets2 = [(torch.randn(T, (2 * heads + nkv) * hd, device=dev).to(bf), t[1], t[2], t[3]) for t in sets]
    qw, kw = torch.ones(heads * hd, device=dev), torch.ones(nkv * hd, device=dev)
    inv32 = inv64[:32].contiguous()
    ms = _timed([(lambda t=t: k.projection_norm_rope_store(t[0], 0, heads * hd, t[1], t[2], t[3], num_heads=heads, num_kv_heads=nkv,
                                                           head_dim=hd, q_weight=qw, k_weight=kw, eps=1e-6, inv_freq=inv32, rot_dim=64,
                                                           rope_style=1, positions=pos, slots=slots)) for t in sets2])
    mem_row("projection_norm_rope_store_lekilix", ms, T * (heads + nkv) * hd * 2 + T * (heads + 2 * nkv) * hd * 2)
    del sets, sets2
    # ---- sum + norm ------------------------------------------------------------------------------------------------------------
    n = 2048
    w = torch.ones(width, device=dev)
    sets = [(torch.randn(n, width, device=dev), torch.randn(n, width, device=dev).to(bf), torch.randn(n, width, device=dev).to(bf),
             torch.empty(n, width, device=dev, dtype=bf)) for _ in range(8)]
    ms = _timed([(lambda t=t: k.normed_add_rms_norm(t[0], t[1], w, 1e-6, None, w, 1e-6, t[3])) for t in sets])
    mem_row("normed_add_rms_norm", ms, n * width * (4 + 2 + 4 + 2))
    ms = _timed([(lambda t=t: k.add2_rms_norm(t[0], t[1], t[2], w, 1e-6, t[3])) for t in sets])
    mem_row("add2_rms_norm_lekilix", ms, n * width * (4 + 2 + 2 + 4 + 2))
    del sets
    # ---- expert products: softmax over the chosen logits and a shared expert  vs  experts by table ---------------------------------
    E, ff, vocab = 64, 1408, 32768
    parts = {}
    for name, params in (("softmax", {"top": 5, "activation": "silu", "score": "softmax_top", "shared_intermediate_size": ff}),
                         ("table_lekilix", {"top": 6, "activation": "clamped_swish", "limit": 7.0, "score": "table", "vocab_size": vocab})):
        part = RoutedExperts(PartSpec("routed_experts", dict(params, hidden_size=width, num_experts=E, intermediate_size=ff,
                                                             weight_on="output")), bf, dev)
        tensors = {}
        for tn, ts in part.tensors().items():
            if ts.kind == "int":
                tensors[tn] = torch.stack([torch.randperm(E)[:6] for _ in range(vocab)]).to(torch.int32).to(dev)
            else:
                tensors[tn] = torch.randn(*ts.shape, device=dev).to(bf) * (1.0 if tn.startswith("router") else 0.02)
        part.bind(tensors)
        del tensors
        parts[name] = part
    for n in (2048, 8):
        h = torch.randn(n, width, device=dev).to(bf)
        for name, part in parts.items():
            ctx_ = StepContext(Workspace(dev))
            ctx_.tokens = torch.randint(0, vocab, (n,), device=dev).to(torch.int32)
            part.forward(h, ctx_)
            ms = _timed(lambda: part.forward(h, ctx_))
            if n >= 128:
                flop_row(f"expert_feed_forward_{name}_{n}", ms, 2.0 * n * 6 * 3 * ff * width)
            else:
                reached = len(set(ctx_.buf("expert_ids", (n, part.top), torch.int32).flatten().tolist())) + (1 if part.shared is not None else 0)
                mem_row(f"expert_feed_forward_{name}_{n}", ms, reached * 3 * ff * width * 2)
    del parts
    torch.cuda.empty_cache()
    # ---- the decayed scan beside the matrix-memory scan --------------------------------------------------------------------------------
    H, d, dv = heads // 2, 128, 256
    cb = state_columns(d, dv)
    wide = 2 * H * d + 2 * H * dv
    decay = torch.linspace(0.6, 0.999, H, device=dev)
    bias = torch.zeros(2 * H, device=dev)
    zb = torch.zeros(H * d, device=dev)
    for B, L in ((8, 1), (64, 1), (1, 2048)):
        n = B * L
        cu = torch.arange(0, n + 1, L, dtype=torch.int32, device=dev)
        sl = torch.arange(B, dtype=torch.int32, device=dev)
        sets = [(torch.randn(n, wide, device=dev).to(bf) * 0.5, torch.randn(n, H * d, device=dev), torch.zeros(B, H, dv // 16, 16, d, device=dev),
                 torch.empty(n, H * dv, device=dev)) for _ in range(4 if L == 1 else 1)]
        for tag, kw in (("head", {"head_decay": decay, "activation": "silu"}), ("channel", {"z_bias": zb, "tau": 16.0, "activation": None})):
            ms = _timed([(lambda t=t: k.decay_scan(t[0], 0, H * d, 2 * H * d, t[2], cu, sl, t[3], num_heads=H, dim=d, v_dim=dv, q_scale=1.0,
                                                   max_q_len=L, **(dict(kw, z=t[1]) if tag == "channel" else kw))) for t in sets])
            if L == 1:
                mem_row(f"decay_scan_{tag}_decode_{B}", ms, B * 2 * H * d * dv * 4)
            else:
                flop_row(f"decay_scan_{tag}_prefill_{L}", ms, 4.0 * L * H * d * dv)
        del sets
        sets = [(torch.randn(n, wide, device=dev).to(bf) * 0.5, torch.randn(n, 2 * H, device=dev),
                 torch.zeros(B, H, dv // cb, state_block_floats(d, cb), device=dev), torch.empty(n, H * dv, device=dev))
                for _ in range(4 if L == 1 else 1)]
        ms = _timed([(lambda t=t: k.matrix_memory_scan(t[0], 0, H * d, 2 * H * d, t[1], bias, t[2], cu, sl, t[3], num_heads=H, dim=d,
                                                       v_dim=dv, columns=cb, cap=15.0, q_scale=d ** -0.5, max_q_len=L)) for t in sets])
        if L == 1:
            mem_row(f"memory_scan_lekilix_decode_{B}", ms, B * 2 * H * (d * dv + d) * 4)
        else:
            flop_row(f"memory_scan_lekilix_prefill_{L}", ms, 4.0 * L * H * d * (dv + 1))
            gate = sets[0][0][:, 2 * H * d + H * dv:]
            wn = torch.ones(H * dv, device=dev)
            o16 = torch.empty(n, H * dv, device=dev, dtype=bf)
            ms = _timed([lambda: k.head_norm_gate_act(sets[0][3], wn, gate, o16, num_heads=1, eps=1e-6, gate_act="sigmoid")] * 4)
            mem_row("norm_over_all_heads_gate", ms, n * H * dv * (4 + 2 + 2))
            ms = _timed([lambda: k.head_norm_gate(sets[0][3], wn, gate, o16, num_heads=H, eps=1e-6)] * 4)
            mem_row("head_norm_gate_lekilix", ms, n * H * dv * (4 + 2 + 2))
        del sets
    k.check_device_status()
    return out


def run_senadra(peaks: dict, width: int = 2048, heads: int = 16) -> dict:
    """The kernels of the Senadra design alone, each beside its like kernel of another path at equal size (16 heads of 128 on
    8 KV heads, chunks of 2,048 positions; recurrences of 16 value heads 128 x 128 on 8 query/key heads; latents of 512 + 64):
      decode attention    8 (and 64) sequences of 4,096 cached tokens, 2,048 of them in the query's chunk: chunked with the
                          distance penalty and the gate  vs  the Qwen3 kernel with a window of 2,048     bytes of cache read
      prefill attention   one sequence of 2,048 tokens (one chunk)  vs  the Qwen3 kernel                 flops of scores and values
      cache write         2,048 tokens: keys, values over their root mean square  vs  per-head norm, rotation, cache write
      sum + norm          2,048 rows: the sum with a factor  vs  the plain sum; the normalised addend (no like kernel)
      feed-forward        2,048 (and 8) rows: up, xIELU, down  vs  gate/up with SwiGLU, down, of equal weights
      delta-rule scan     8 / 64 sequences of one token (bytes of state) and one sequence of 2,048 tokens  vs  the
                          matrix-memory scan of equal state (8 heads 128 x 256)
    """
    import torch
    from .. import ops
    from ..parts.matrix_memory import state_block_floats, state_columns
    k = ops.kernels()
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    nkv, hd, page, chunk = 8, 128, 16, 2048
    out = {}
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]

    def mem_row(name, ms, nbytes):
        out[name] = {"ms": ms, "gb_s": nbytes / ms / 1e6, "of_hbm_peak": nbytes / ms / 1e6 / hbm}

    def flop_row(name, ms, flops):
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "of_bf16_peak": flops / ms / 1e9 / tfl}

    r1 = torch.rand(heads, device=dev) * 0.3
    r2 = torch.rand(heads, device=dev) + 0.5
    # ---- decode attention ------------------------------------------------------------------------------------------------
    for B, ctx in ((8, 4096), (64, 4096)):
        meta, pages = _meta([ctx] * B, [1] * B, page, dev)
        copies = [(torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3, torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3)
                  for _ in range(3 if B == 8 else 2)]
        q = torch.randn(B, heads * hd, device=dev).to(bf) * 0.1
        gate = torch.randn(B, heads * hd, device=dev).to(bf)
        o = torch.empty(B, heads * hd, device=dev, dtype=bf)
        nbytes = B * (ctx - chunk) * 2 * nkv * hd * 2
        ms = _timed([(lambda c=c: k.chunked_attention(q, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, k_dim=hd, v_dim=hd,
                                                      scale=0.088, chunk=chunk, window=None, r1=r1, r2=r2, gate=gate)) for c in copies])
        mem_row(f"decode_attention_chunked_{B}x{ctx}", ms, nbytes)
        q3 = q.view(B, heads, hd)
        ms = _timed([(lambda c=c: k.paged_attention(q3, c[0], c[1], o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088,
                                                    window=chunk)) for c in copies])
        mem_row(f"decode_attention_qwen3_{B}x{ctx}", ms, nbytes)
        del copies
    torch.cuda.empty_cache()
    # ---- prefill attention -----------------------------------------------------------------------------------------------
    T = 2048
    meta, pages = _meta([T], [T], page, dev)
    kc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    vc = torch.randn(pages, nkv, page, hd, device=dev).to(bf) * 0.3
    q = torch.randn(T, heads * hd, device=dev).to(bf) * 0.1
    gate = torch.randn(T, heads * hd, device=dev).to(bf)
    o = torch.empty(T, heads * hd, device=dev, dtype=bf)
    pairs = T * (T + 1) / 2
    ms = _timed([lambda: k.chunked_attention(q, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, k_dim=hd, v_dim=hd, scale=0.088,
                                             chunk=chunk, window=None, r1=r1, r2=r2, gate=gate)] * 4)
    flop_row("prefill_attention_chunked", ms, 4.0 * heads * hd * pairs)
    q3 = q.view(T, heads, hd)
    ms = _timed([lambda: k.paged_attention(q3, kc, vc, o, meta, num_heads=heads, num_kv_heads=nkv, head_dim=hd, scale=0.088, window=None)] * 4)
    flop_row("prefill_attention_qwen3", ms, 4.0 * heads * hd * pairs)
    # ---- cache write -----------------------------------------------------------------------------------------------------
    slots = torch.arange(T, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    front = 2 * heads * hd
    sets = [(torch.randn(T, front + 2 * nkv * hd, device=dev).to(bf), torch.zeros_like(kc), torch.zeros_like(vc)) for _ in range(4)]
    ms = _timed([(lambda t=t: k.kv_store_normed(t[0], front, front + nkv * hd, t[1], t[2], slots, num_kv_heads=nkv, k_dim=hd, v_dim=hd,
                                                eps=1e-6, norm_values=True)) for t in sets])
    mem_row("kv_store_normed", ms, 2 * T * 2 * nkv * hd * 2)
    sets2 = [(torch.randn(T, (heads + 2 * nkv) * hd, device=dev).to(bf), torch.empty(T, heads, hd, device=dev, dtype=bf), t[1], t[2])
             for t in sets]
    qw2, kw2 = torch.ones(hd, device=dev), torch.ones(hd, device=dev)
    inv_full = torch.pow(torch.tensor(500000.0), -torch.arange(hd // 2, dtype=torch.float32) / (hd // 2)).to(dev)
    ms = _timed([(lambda t=t: k.qk_norm_rope_store(t[0], t[1], t[2], t[3], num_heads=heads, num_kv_heads=nkv, head_dim=hd, q_weight=qw2,
                                                   k_weight=kw2, eps=1e-6, inv_freq=inv_full, rot_dim=hd, rope_style=0, positions=pos,
                                                   slots=slots, write_kv=True)) for t in sets2])
    mem_row("qk_norm_rope_store_qwen3", ms, 2 * T * (heads + 2 * nkv) * hd * 2)
    del sets, sets2, kc, vc
    # ---- sums and norms ---------------------------------------------------------------------------------------------------
    n = 2048
    w = torch.ones(width, device=dev)
    sets = [(torch.randn(n, width, device=dev), torch.randn(n, width, device=dev).to(bf), torch.empty(n, width, device=dev, dtype=bf))
            for _ in range(8)]
    ms = _timed([(lambda t=t: k.scaled_add_rms_norm(t[0], t[1], 0.5, w, 1e-6, t[2])) for t in sets])
    mem_row("scaled_add_rms_norm", ms, n * width * (4 + 2 + 4 + 2))
    ms = _timed([(lambda t=t: k.add_rms_norm(t[0], t[1], w, 1e-6, t[2])) for t in sets])
    mem_row("add_rms_norm_qwen3", ms, n * width * (4 + 2 + 4 + 2))
    ms = _timed([(lambda t=t: k.scaled_add_unit_rms(t[0], t[1], 0.5, w, 1e-6)) for t in sets])
    mem_row("scaled_add_unit_rms", ms, n * width * (4 + 2 + 4))
    del sets
    # ---- feed-forward: ungated with xIELU beside gated with SwiGLU, equal weights -------------------------------------------
    from ..config.spec import PartSpec
    from ..engine.runner import StepContext, Workspace
    from ..parts.mlp import PlainMLP
    inter = 4 * width
    for n in (2048, 8):
        h = torch.randn(n, width, device=dev).to(bf)
        reps = 3 if n < 128 else 1
        plain_parts = []
        for _ in range(reps):
            part = PlainMLP(PartSpec("plain_mlp", {"hidden_size": width, "intermediate_size": inter * 3 // 2, "activation": "xielu"}), bf, dev)
            part.bind({"up": torch.randn(inter * 3 // 2, width, device=dev).to(bf) * 0.02,
                       "down": torch.randn(width, inter * 3 // 2, device=dev).to(bf) * 0.02, "act": torch.tensor([0.3, -0.2], device=dev)})
            plain_parts.append(part)
        ctx_ = StepContext(Workspace(dev))
        ms = _timed([(lambda p_=p_: p_.forward(h, ctx_)) for p_ in plain_parts] * (1 if n < 128 else 3))
        wgus = [torch.randn(2 * inter, width, device=dev).to(bf) * 0.02 for _ in range(reps)]
        wds = [torch.randn(width, inter, device=dev).to(bf) * 0.02 for _ in range(reps)]
        a2, y2 = torch.empty(n, inter, device=dev, dtype=bf), torch.empty(n, width, device=dev, dtype=bf)
        gu = torch.empty(n, 2 * inter, device=dev, dtype=bf)
        fused = k.can_fuse_swiglu(h, wgus[0], 8)

        def dense_on(wa, wb):
            def run_():
                if fused:
                    k.linear_swiglu(h, wa, a2)
                else:
                    k.linear(h, wa, gu)
                    k.swiglu(gu, a2, 8)
                k.linear(a2, wb, y2)
            return run_
        ms_dense = _timed([dense_on(a, b) for a, b in zip(wgus, wds)] * (1 if n < 128 else 3))
        if n >= 128:
            flop_row(f"xielu_feed_forward_{n}", ms, 2.0 * n * 3 * inter * width)
            flop_row(f"swiglu_feed_forward_{n}", ms_dense, 2.0 * n * 3 * inter * width)
        else:
            mem_row(f"xielu_feed_forward_{n}", ms, 3 * inter * width * 2)
            mem_row(f"swiglu_feed_forward_{n}", ms_dense, 3 * inter * width * 2)
        del plain_parts, wgus, wds
    torch.cuda.empty_cache()
    # ---- the delta-rule scan beside the matrix-memory scan of equal state ------------------------------------------------------
    H, G, d, dv, taps = heads, heads // 2, 128, 128, 4
    channels = 2 * G * d + H * dv
    conv_w = torch.randn(channels, taps, device=dev) * 0.3
    a_log, dt_bias = torch.zeros(H, device=dev), torch.zeros(H * d, device=dev)
    n_state = k.delta_state_floats(H, G, d, dv, taps)
    ws = Workspace(dev)
    for B, L in ((8, 1), (64, 1), (1, 2048)):
        n = B * L
        sets = [(torch.randn(n, channels + H, device=dev).to(bf) * 0.5, torch.randn(n, H * d, device=dev),
                 torch.zeros(B, n_state, device=dev), torch.empty(n, H * dv, device=dev)) for _ in range(4 if L == 1 else 1)]
        sc = StepContext(ws)
        sc.cu_q = torch.arange(0, n + 1, L, dtype=torch.int32, device=dev)
        sc.state_slots = torch.arange(B, dtype=torch.int32, device=dev)
        sc.seq_of_token = torch.arange(n, dtype=torch.int32, device=dev) // L
        ms = _timed([(lambda t=t: k.delta_rule(t[0], 0, channels, t[1], conv_w, a_log, dt_bias, t[2], sc, t[3], num_heads=H,
                                               num_kv_heads=G, dim=d, v_dim=dv)) for t in sets])
        if L == 1:
            mem_row(f"delta_rule_decode_{B}", ms, B * 2 * H * d * dv * 4)
        else:
            flop_row(f"delta_rule_prefill_{L}", ms, 6.0 * L * H * d * dv)
        del sets
        Hm, dm, dvm, cap = heads // 2, 128, 256, 15.0
        cb = state_columns(dm, dvm)
        wide = 2 * Hm * dm + 2 * Hm * dvm
        bias = torch.zeros(2 * Hm, device=dev)
        sets = [(torch.randn(n, wide, device=dev).to(bf) * 0.5, torch.randn(n, 2 * Hm, device=dev),
                 torch.zeros(B, Hm, dvm // cb, state_block_floats(dm, cb), device=dev), torch.empty(n, Hm * dvm, device=dev))
                for _ in range(4 if L == 1 else 1)]
        ms = _timed([(lambda t=t: k.matrix_memory_scan(t[0], 0, Hm * dm, 2 * Hm * dm, t[1], bias, t[2], sc.cu_q, sc.state_slots, t[3],
                                                       num_heads=Hm, dim=dm, v_dim=dvm, columns=cb, cap=cap, q_scale=dm ** -0.5,
                                                       max_q_len=L)) for t in sets])
        if L == 1:
            mem_row(f"memory_scan_decode_{B}", ms, B * 2 * Hm * (dm * dvm + dm) * 4)
        else:
            flop_row(f"memory_scan_prefill_{L}", ms, 4.0 * L * Hm * dm * (dvm + 1))
        del sets
    k.check_device_status()
    return out


def main(argv=None) -> int:
    from . import workloads
    peaks, kind = workloads.load_peaks()
    print(json.dumps({"peaks": dict(peaks, kind=kind), "kernels": run(peaks)}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
