"""Time one kernel of the engine in isolation, on the device clock, against its roofline.

    python -m edgerag_b200.ops.microbench decode-attention --batch 8 --context 8192
    python -m edgerag_b200.ops.microbench prefill-attention --tokens 2048
    python -m edgerag_b200.ops.microbench linear --m 8 --n 6144 --k 2048
    python -m edgerag_b200.ops.microbench latent-attention --batch 8 --context 8192
    python -m edgerag_b200.ops.microbench ssm-scan --batch 8 --tokens 1
    python -m edgerag_b200.ops.microbench step-kernels --layers 4 --batch 8 --context 8192 --iters 4

Each case builds random inputs larger than the 126 MB L2 where the real workload is (or says that
it is not), runs warm-up launches, then times ``--iters`` launches replayed from one CUDA graph with
CUDA events and prints one JSON line with the median per launch.  Fractions are of the peaks in a
JSON file ``{"hbm_gbs": ..., "bf16_tflops": ...}`` named by ``--peaks`` or, by default,
``MEASURED_PEAKS.json`` in the working directory or beside the package; without such a file they
are of the stated defaults, and the line says which (``"peaks"``).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

from . import kernels

HBM_GBS, BF16_TFLOPS = 6650.0, 1590.0   # defaults (a B200's copy bandwidth and library bf16 product rate) when no file is found
PEAKS_FROM = "defaults"


def load_peaks(path: str | None) -> None:
    """Take the roofline denominators from a JSON file of measured peaks, if there is one."""
    global HBM_GBS, BF16_TFLOPS, PEAKS_FROM
    candidates = [Path(path)] if path else [Path.cwd() / "MEASURED_PEAKS.json",
                                            Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"]
    for cand in candidates:
        try:
            raw = json.loads(cand.read_text())
            HBM_GBS, BF16_TFLOPS, PEAKS_FROM = float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), f"measured ({cand.name})"
            return
        except (OSError, KeyError, ValueError):
            continue
    if path:
        raise SystemExit(f"--peaks {path}: not a JSON file with hbm_gbs and bf16_tflops")


def _time(fn, iters: int, warmup: int, rounds: int = 5) -> float:
    """Median over ``rounds`` of the time per launch of ``iters`` launches, in microseconds.  The launches
    are captured into one CUDA graph and replayed, so that kernels of a few microseconds are timed
    back to back as they run inside a step, not at the rate the host can issue them."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / iters)
    return statistics.median(times)


def _paged(batch: int, context: int, nkv: int, d: int, page: int, dtype, shuffle: bool = True):
    """Key and value pools of ``batch`` sequences of ``context`` tokens with their block tables."""
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    kp = torch.randn((n_pages, nkv, page, d), device="cuda", dtype=torch.float32).to(dtype)
    vp = torch.randn((n_pages, nkv, page, d), device="cuda", dtype=torch.float32).to(dtype)
    order = torch.randperm(n_pages) if shuffle else torch.arange(n_pages)
    tables = order.view(batch, pages_per).to(torch.int32).cuda()
    return kp, vp, tables


def decode_attention(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    window, keep, chunk = getattr(a, "window", 0), getattr(a, "keep_first", 0), getattr(a, "chunk", 0)
    seen = min(a.context, window + keep) if window > 0 else a.context       # keys a query reads
    if chunk > 0:           # the query is the context's last position: it reads its chunk up to itself
        seen = (a.context - 1) % chunk + 1
    nbytes = 2 * a.batch * seen * a.kv_heads * a.head_dim * (2 if dtype == torch.bfloat16 else 4)
    # --cold: rotate over so many caches that each launch finds its keys and values in DRAM, as a
    # step does whose weights have passed through L2 since the layer's cache was last read
    reps = max(2, int(300e6 // nbytes) + 1) if a.cold else 1
    caches = [_paged(a.batch, a.context, a.kv_heads, a.head_dim, a.page, dtype, not a.sequential_pages) for _ in range(reps)]
    state = {"i": 0}

    def cache():
        state["i"] = (state["i"] + 1) % reps
        return caches[state["i"]]

    q = torch.randn((a.batch, a.heads * a.head_dim), device="cuda").to(dtype)
    out = torch.empty_like(q)
    pos = torch.full((a.batch,), a.context - 1, dtype=torch.int32, device="cuda")
    tok = torch.arange(a.batch, dtype=torch.int32, device="cuda")
    if a.split <= 0:        # as the engine chooses it: from the batch and a power-of-two bound on the context
        bound, granule = kernels.context_bound(-(-a.context // a.page))
        if window > 0 or chunk > 0:
            bound = min(bound, -(-(window + keep + chunk) // a.page))
            granule = bound
        a.split, heads = kernels.choose_decode_plan(a.batch, a.kv_heads, bound * a.page, a.page, a.head_dim, a.kernel != "bulk",
                                                    granule * a.page)
        a.head_group = a.head_group or heads
    splits = (a.context - 1) // a.split + 1
    if window > 0 or chunk > 0:
        splits = min(splits, (window + chunk) // a.split + 2)
    acc_n, ml_n = kernels.decode_scratch_floats(a.batch, a.heads, a.head_dim, splits)
    acc, ml = torch.empty(acc_n, device="cuda"), torch.empty(ml_n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = a.head_dim ** -0.5
    if a.kernel == "gqa":
        fn = lambda: kernels.attention_decode_gqa(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                                  status, split_keys=a.split, window=window, keep_first=keep, chunk=chunk)
    elif a.kernel == "bulk":
        fn = lambda: kernels.attention_decode_bulk(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                                   status, split_keys=a.split, head_group=a.head_group, window=window, keep_first=keep,
                                                   chunk=chunk)
    else:
        fn = lambda: kernels.attention_decode(q, *cache(), tok, pos, out, a.heads, scale, acc, ml, splits,  # noqa: E731
                                              split_keys=a.split, window=window, keep_first=keep, chunk=chunk)
    us = _time(fn, max(a.iters, 2 * reps), a.warmup)
    return {"case": "decode-attention", "kernel": a.kernel, "split": a.split, "head_group": a.head_group, "us": round(us, 2),
            "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4),
            "status": int(status), "from_dram": bool(a.cold) or nbytes > 126e6, "window": window, "keep_first": keep, "chunk": chunk}


def prefill_attention(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    total = a.past + a.tokens
    kp, vp, tables = _paged(1, total, a.kv_heads, a.head_dim, a.page, dtype, not a.sequential_pages)
    width = (a.heads + 2 * a.kv_heads) * a.head_dim
    qkv = torch.randn((a.tokens, width), device="cuda").to(dtype)
    out = torch.empty((a.tokens, a.heads * a.head_dim), device="cuda", dtype=dtype)
    pos = torch.arange(a.past, total, dtype=torch.int32, device="cuda")
    starts = torch.tensor([0, a.tokens], dtype=torch.int32, device="cuda")
    seq_of = torch.zeros(a.tokens, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = a.head_dim ** -0.5
    window, keep, chunk = getattr(a, "window", 0), getattr(a, "keep_first", 0), getattr(a, "chunk", 0)
    if a.kernel == "tc":
        blocks = kernels.prefill_tc_blocks([a.tokens])
        reach = min(total, window + keep + chunk + kernels.PREFILL_TC_ROWS) if window > 0 or chunk > 0 else total
        ranges = a.key_splits or kernels.prefill_tc_key_splits(blocks, a.heads, reach, qkv.device)
        need_o, need_ml = kernels.prefill_tc_scratch_floats(a.tokens, a.heads, ranges)
        part_o, part_ml = torch.empty(need_o, device="cuda"), torch.empty(need_ml, device="cuda")
        fn = lambda: kernels.attention_prefill_tc(qkv, kp, vp, tables, starts, pos, out, blocks, a.heads, scale, status,  # noqa: E731
                                                  key_splits=ranges, part_o=part_o, part_ml=part_ml, window=window, keep_first=keep,
                                                  chunk=chunk)
    else:
        fn = lambda: kernels.attention_rows(qkv, kp, vp, tables, seq_of, pos, out, a.heads, scale, window=window,  # noqa: E731
                                            keep_first=keep, chunk=chunk)
    us = _time(fn, a.iters, a.warmup)
    if window > 0:      # (query, key) pairs that are seen: the window's keys and the kept ones before it
        p = torch.arange(a.past, total, dtype=torch.float64)
        lo = (p - window + 1).clamp_min(0)
        pairs = float((p - lo + 1 + torch.minimum(lo, torch.tensor(float(keep)))).sum())
    elif chunk > 0:     # every query sees the keys of its own chunk up to itself
        p = torch.arange(a.past, total, dtype=torch.float64)
        pairs = float((p % chunk + 1).sum())
    else:
        pairs = a.tokens * a.past + a.tokens * (a.tokens + 1) / 2
    flops = 4.0 * a.heads * a.head_dim * pairs
    return {"case": "prefill-attention", "kernel": a.kernel, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
            "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4), "status": int(status), "window": window, "keep_first": keep, "chunk": chunk}


def linear(a) -> dict:
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    reps = max(1, int(200e6 // (a.n * a.k * 2)) + 1)    # rotate over several weight copies: more than L2 in total
    ws = [torch.randn((a.n, a.k), device="cuda").to(dtype) for _ in range(reps)]
    x = torch.randn((a.m, a.k), device="cuda").to(dtype)
    out = torch.empty((a.m, a.n), device="cuda", dtype=torch.float32 if a.out32 else dtype)
    out_glu = torch.empty((a.m, a.n // 2), device="cuda", dtype=dtype) if a.glu else None
    n_parts = kernels.linear_parts_slices(ws[0]) if a.parts else 0
    parts = torch.empty((n_parts, a.m, a.n), device="cuda", dtype=torch.float32) if n_parts else None
    state = {"i": 0}

    def fn():
        state["i"] = (state["i"] + 1) % reps
        if a.parts:
            kernels.linear_parts(x, ws[state["i"]], parts)
        elif a.tc:
            (kernels.linear_tc_glu if a.glu else kernels.linear_tc)(x, ws[state["i"]], out_glu if a.glu else out)
        elif a.glu:
            kernels.linear_glu(x, ws[state["i"]], out_glu)
        else:
            kernels.linear(x, ws[state["i"]], out, library=a.library)

    us = _time(fn, a.iters, a.warmup)
    nbytes = a.n * a.k * x.element_size() + a.m * a.k * x.element_size() + out.numel() * out.element_size()
    flops = 2.0 * a.m * a.n * a.k
    if n_parts:
        nbytes += parts.numel() * 4 - out.numel() * out.element_size()
    return {"case": "linear", "m": a.m, "n": a.n, "k": a.k, "library": bool(a.library), "tc": bool(a.tc), "glu": bool(a.glu), "parts": n_parts, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
            "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4), "tflops": round(flops / us / 1e6, 2)}


def step_kernels(a) -> dict:
    """Which kernels a step's time goes to: the SmolVLM-2.2B layer sizes with ``--layers`` layers (or the
    model of ``a.config``, a config.json as a dict, with ``a.vocab``), a
    prefill of ``--tokens`` tokens and decode steps of ``--batch`` sequences at ``--context``, run
    eagerly under the CUDA activity tracer without chained launches (so that a kernel's time is its
    own).  The microseconds are per launch and carry the tracer's overhead: read them as shares."""
    import os

    os.environ["EDGERAG_B200_NO_CHAIN"] = "1"          # read when the first library launches a kernel
    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine, EngineOptions
    from ..engine.step import StepEntry

    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": a.layers, "hidden_size": 2048,
           "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": 64, "intermediate_size": 8192,
           "vocab_size": 49155, "rope_theta": 273768.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "hidden_act": "silu", "max_position_embeddings": 8192, "pad_token_id": 0}
    if getattr(a, "config_json", None):       # any model: a config.json (its vocabulary size is searched under the usual keys)
        with open(a.config_json) as f:
            cfg = json.load(f)
    cfg = getattr(a, "config", None) or cfg
    vocab = getattr(a, "vocab", None) or cfg.get("vocab_size") or cfg.get("vocab") or 49155
    rows_shown = getattr(a, "rows", None) or 12
    eng = Engine.from_config(cfg, 0, 0.02, EngineOptions(
        dtype="bfloat16", block_size=16, num_blocks=a.batch * (a.context // 16 + 2) + a.tokens // 16 + 64,
        max_batch_size=a.batch + 2, chunk_size=a.tokens, max_step_tokens=a.tokens + a.batch, max_model_len=a.context + 8,
        cuda_graphs=False))
    r = eng.runner
    ids = torch.randint(0, vocab, (a.tokens,)).tolist()

    def table(prof, launches_of):
        rows = [(e.key, e.device_time_total / max(1, e.count), e.count) for e in prof.key_averages() if e.device_time_total > 0]
        total = sum(us * n for _, us, n in rows)
        rows.sort(key=lambda x: -x[1] * x[2])
        return {"total_us_per_" + launches_of[0]: round(total / launches_of[1], 1),
                "kernels": [{"name": k[:70], "us": round(us, 2), "calls": n, "share": round(us * n / total, 3)} for k, us, n in rows[:rows_shown]]}

    def prefill(name):
        r.admit(name)
        r.step([StepEntry(name, tokens=ids, want=[a.tokens - 1])])
        r.release(name)

    prefill("w0")
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as p1:
        prefill("w1")
        torch.cuda.synchronize()
    names = [f"d{i}" for i in range(a.batch)]
    for n in names:
        r.admit(n)
        eng.cache.grow(n, a.context - 64)
        eng.cache.advance(n, a.context - 64)
    for _ in range(3):
        r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as p2:
        for _ in range(a.iters):
            r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])
        torch.cuda.synchronize()
    return {"case": "step-kernels", "layers": a.layers, "batch": a.batch, "context": a.context, "tokens": a.tokens,
            "prefill": table(p1, ("step", 1)), "decode": table(p2, ("step", a.iters))}


def step_timeline(a) -> dict:
    """Where a decode step's time goes when its kernels run as they do in serving: replayed from a CUDA
    graph with chained launches, so that a kernel starts while the one before it drains.  The activity
    tracer gives every kernel's start and end; a kernel's share of the critical path is the time from
    the end of the kernels before it to its own end.  ``--layers`` layers of the SmolVLM-2.2B sizes,
    ``--batch`` sequences at ``--context``; averages over the layers after the first, in microseconds
    (they carry the tracer's overhead: read them as shares)."""
    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine, EngineOptions
    from ..engine.step import StepEntry

    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": a.layers, "hidden_size": 2048,
           "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": 64, "intermediate_size": 8192,
           "vocab_size": 49155, "rope_theta": 273768.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "hidden_act": "silu", "max_position_embeddings": 8192, "pad_token_id": 0}
    eng = Engine.from_config(cfg, 0, 0.02, EngineOptions(
        dtype="bfloat16", block_size=16, num_blocks=a.batch * (a.context // 16 + 2) + 64, max_batch_size=a.batch + 2,
        max_step_tokens=512 + a.batch, max_model_len=a.context + 8, cuda_graphs=True))
    r = eng.runner
    names = [f"d{i}" for i in range(a.batch)]
    for n in names:
        r.admit(n)
        eng.cache.grow(n, a.context - 16)
        eng.cache.advance(n, a.context - 16)
    step = lambda: r.step([StepEntry(n, tokens=[5], want=[0]) for n in names])  # noqa: E731
    for _ in range(4):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if "cuda" in str(e.device_type).lower() and "Memcpy" not in e.name),
                    key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(events) if "embed_rows" in e.name)
    events = events[first:]
    names_of = [e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:48] for e in events]
    norms = [i for i, n in enumerate(names_of) if n.startswith("add_rmsnorm")]
    per_layer = norms[2] - norms[0] if len(norms) > 2 else len(events) - 1      # a layer: from its first norm to the next layer's
    t0, frontier = events[0].time_range.start, events[0].time_range.end
    shares: dict[tuple[int, str], list[float]] = {}
    starts = []
    for i, e in enumerate(events[1: 1 + per_layer * a.layers]):
        if i % per_layer == 0:
            starts.append(e.time_range.start)
        name = names_of[1 + i]
        shares.setdefault((i % per_layer, name), []).append(max(0.0, e.time_range.end - max(frontier, e.time_range.start)))
        frontier = max(frontier, e.time_range.end)
    rows = [{"kernel": name, "critical_us": round(sum(v[1:]) / max(1, len(v) - 1), 2)} for (_, name), v in sorted(shares.items())]
    period = (starts[-1] - starts[0]) / max(1, len(starts) - 1) if len(starts) > 1 else 0.0
    return {"case": "step-timeline", "layers": a.layers, "batch": a.batch, "context": a.context, "replayed_from_graph": r.graph_replays > 0,
            "layer_period_us": round(period, 2), "step_us": round(events[-1].time_range.end - t0, 1), "kernels_of_a_layer": rows}


def latent_attention(a) -> dict:
    """The attention kernel over cache rows [c | kr]: single tokens at the end of ``context`` cached tokens
    (bound by the rows it reads), or ``tokens`` prompt tokens after ``past`` (bound by its products)."""
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    dk, item = a.rank + a.rot, 2 if dtype == torch.bfloat16 else 4
    decode = a.tokens <= 0
    n_seqs = a.batch if decode else 1
    total = a.context if decode else a.past + a.tokens
    n = n_seqs if decode else a.tokens
    pages_per = -(-total // a.page)
    reps = max(2, int(300e6 // (n_seqs * total * dk * item)) + 1) if (decode and a.cold) else 1
    pools = [torch.randn((n_seqs * pages_per, 1, a.page, dk), device="cuda").to(dtype) for _ in range(reps)]
    tables = torch.randperm(n_seqs * pages_per).to(torch.int32).view(n_seqs, pages_per).cuda()
    q = torch.randn((n, a.heads, dk), device="cuda") * dk ** -0.5
    out = torch.empty((n, a.heads, a.rank), device="cuda", dtype=dtype)
    if decode:
        pos = torch.full((n,), total - 1, dtype=torch.int32, device="cuda")
        seq_of = torch.arange(n, dtype=torch.int32, device="cuda")
        blocks = -(-n * a.heads // 4)
        want = max(1, min(-(-2 * kernels._sms(q.device) // blocks), -(-total // 64), kernels.LATENT_MAX_SPLITS))
        split = a.split or -(-(-(-total // want)) // 64) * 64
        n_splits = -(-total // split)
    else:
        pos = torch.arange(a.past, total, dtype=torch.int32, device="cuda")
        seq_of = torch.zeros(n, dtype=torch.int32, device="cuda")
        split, n_splits = 0, 1
    window = int(getattr(a, "window", 0) or 0)
    reach = min(total, window) if window else total          # keys a single token reads
    if decode and window and not a.split:
        want = max(1, min(-(-2 * kernels._sms(q.device) // blocks), -(-reach // 64), kernels.LATENT_MAX_SPLITS))
        split = -(-(-(-reach // want)) // 64) * 64
        n_splits = min(-(-total // split), (window - 1) // split + 2)
    part = torch.empty(max(1, kernels.latent_scratch_floats(n, a.heads, a.rank, n_splits)), device="cuda")
    state = {"i": 0}

    mma = a.kernel == "mma" and kernels.latent_mma_supported(dtype, a.rank, a.rot)
    if mma:
        mt = 2 if (not decode or a.heads > 16) else 1
        q_lens = [1] * n if decode else [a.tokens]
        tiles = kernels.latent_mma_tiles(q_lens, a.heads, mt)
        starts = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
        if decode and not a.split:
            want = max(1, min(-(-kernels._sms(q.device) // tiles), -(-reach // 64), kernels.LATENT_MAX_SPLITS))
            split = -(-(-(-reach // want)) // 64) * 64
            n_splits = -(-total // split) if not window else min(-(-total // split), (window - 1) // split + 2)
            part = torch.empty(max(1, kernels.latent_scratch_floats(n, a.heads, a.rank, n_splits)), device="cuda")

    def fn():
        state["i"] = (state["i"] + 1) % reps
        if mma:
            kernels.latent_attention_mma(q, pools[state["i"]], tables, starts, pos, out, 1.0, 0, n_seqs, 0, n, tiles, mt,
                                         split_keys=split, n_splits=n_splits, part=part if n_splits > 1 else None, window=window)
        else:
            kernels.latent_attention(q, pools[state["i"]], tables, seq_of, pos, out, 1.0, 0, n, split_keys=split,
                                     n_splits=n_splits, part=part if n_splits > 1 else None, window=window)

    us = _time(fn, max(a.iters, 2 * reps), a.warmup)
    nbytes = n_seqs * reach * dk * item
    pairs = n * reach if decode else _seen_pairs(a.tokens, a.past, window)
    flops = 2.0 * a.heads * (dk + a.rank) * pairs
    return {"case": "latent-attention", "kernel": "mma" if mma else "general", "mode": "decode" if decode else "prefill", "splits": n_splits, "us": round(us, 2),
            "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4),
            "tflops": round(flops / us / 1e6, 2), "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4),
            "from_dram": bool(decode and (a.cold or nbytes > 126e6))}


def _seen_pairs(tokens: int, past: int, window: int) -> float:
    """(query, key) pairs that ``tokens`` queries after ``past`` cached tokens see, under a window or without one."""
    if not window:
        return tokens * past + tokens * (tokens + 1) / 2
    return float(sum(min(window, past + i + 1) for i in range(tokens)))


def diff_attention(a) -> dict:
    """The differential-attention kernel: single tokens at the end of ``context`` cached tokens (bound by the keys and
    values of their windows), or ``tokens`` prompt tokens after ``past`` (bound by its arithmetic: per seen pair and
    head, two score products of ``dim`` and two value sums of ``vdim``)."""
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    item = 2 if dtype == torch.bfloat16 else 4
    H, G, d, dv, window = a.heads, a.kv_heads, a.dim, a.vdim, int(a.window or 0)
    decode = a.tokens <= 0
    n_seqs = a.batch if decode else 1
    total = a.context if decode else a.past + a.tokens
    n = n_seqs if decode else a.tokens
    pages_per = -(-total // a.page)
    reach = min(total, window) if window else total
    reps = max(2, int(300e6 // (n_seqs * reach * G * (2 * d + dv) * item)) + 1) if (decode and a.cold) else 1
    kp = [torch.randn((n_seqs * pages_per, G, a.page, 2 * d), device="cuda").to(dtype) for _ in range(reps)]
    vp = [torch.randn((n_seqs * pages_per, G, a.page, dv), device="cuda").to(dtype) for _ in range(reps)]
    tables = torch.randperm(n_seqs * pages_per).to(torch.int32).view(n_seqs, pages_per).cuda()
    q = (torch.randn((n, H * 2 * d), device="cuda") * d ** -0.5).to(dtype)
    out = torch.empty((n, H * dv), device="cuda", dtype=dtype)
    split, n_splits = 0, 1
    if decode:
        pos = torch.full((n,), total - 1, dtype=torch.int32, device="cuda")
        seq_of = torch.arange(n, dtype=torch.int32, device="cuda")
        blocks = -(-n * H // 4)
        want = max(1, min(-(-2 * kernels._sms(q.device) // blocks), -(-reach // 64), 64))
        split = a.split or -(-(-(-reach // want)) // 64) * 64
        n_splits = -(-total // split) if not window else min(-(-total // split), (window - 1) // split + 2)
    else:
        pos = torch.arange(a.past, total, dtype=torch.int32, device="cuda")
        seq_of = torch.zeros(n, dtype=torch.int32, device="cuda")
    mma = getattr(a, "kernel", "mma") == "mma" and kernels.diff_mma_supported(dtype, d, dv)
    if mma:
        q_lens = [1] * n if decode else [a.tokens]
        tile_rows = (8 if H // G <= 8 else 16 if H // G <= 16 else 64) if decode else 64
        tiles = kernels.diff_mma_tiles(q_lens, H // G, tile_rows)
        starts = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
        if decode and not a.split:      # as the mixer plans: a block per (sequence, kv head, split)
            want = max(1, min(-(-2 * kernels._sms(q.device) // max(1, n * G)), -(-reach // 64), 64))
            split = -(-(-(-reach // want)) // 64) * 64
            n_splits = -(-total // split) if not window else min(-(-total // split), (window - 1) // split + 2)
    part = torch.empty(max(1, n * H * n_splits * kernels.diff_part_floats(dv)), device="cuda")
    state = {"i": 0}

    def fn():
        state["i"] = (state["i"] + 1) % reps
        if mma:
            kernels.diff_attention_mma(q, kp[state["i"]], vp[state["i"]], tables, starts, pos, out, H, d ** -0.5, 0.3, 1e-6, 0.5, 0,
                                       n_seqs, 0, n, tiles, window=window, softcap=float(a.softcap), split_keys=split,
                                       n_splits=n_splits, part=part if n_splits > 1 else None, tile_rows=tile_rows)
            return
        kernels.diff_attention(q, kp[state["i"]], vp[state["i"]], tables, seq_of, pos, out, H, d ** -0.5, 0.3, 1e-6, 0.5, 0, n,
                               window=window, softcap=float(a.softcap), split_keys=split, n_splits=n_splits,
                               part=part if n_splits > 1 else None)

    us = _time(fn, max(a.iters, 2 * reps), a.warmup)
    nbytes = n_seqs * reach * G * (2 * d + dv) * item
    pairs = n * reach if decode else _seen_pairs(a.tokens, a.past, window)
    flops = 2.0 * H * (2 * d + 2 * dv) * pairs
    return {"case": "diff-attention", "kernel": "mma" if mma else "general", "mode": "decode" if decode else "prefill", "splits": n_splits, "us": round(us, 2),
            "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4),
            "tflops": round(flops / us / 1e6, 2), "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4),
            "from_dram": bool(decode and (a.cold or nbytes > 126e6))}


def ssm_scan(a) -> dict:
    """The recurrence kernel: ``batch`` requests of ``tokens`` tokens each.  One token per request is bound by
    the state it reads and writes; a prompt portion by the walk along its tokens."""
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    inner, ch = a.heads * a.head_dim, a.heads * a.head_dim + 2 * a.groups * a.state
    n = a.batch * a.tokens
    xbc = (torch.randn((n, ch), device="cuda") * 0.3).to(dtype)
    proj = torch.randn((n, a.heads), device="cuda").to(dtype)
    vec = [torch.randn(a.heads, device="cuda") for _ in range(3)]
    state = torch.zeros((a.batch, a.heads, a.state, a.head_dim), device="cuda")
    y = torch.empty((n, inner), device="cuda")
    starts = (torch.arange(a.batch + 1, dtype=torch.int32) * a.tokens).cuda()
    slots = torch.arange(a.batch, dtype=torch.int32).cuda()
    fn = lambda: kernels.ssm_scan(xbc, proj, 0, vec[0], vec[1], vec[2], state, a.batch, starts, slots, y, a.groups)  # noqa: E731
    us = _time(fn, a.iters, a.warmup)
    item = 2 if dtype == torch.bfloat16 else 4
    nbytes = 2 * state.numel() * 4 + n * (ch * item + inner * 4)
    flops = 6.0 * n * a.heads * a.state * a.head_dim
    return {"case": "ssm-scan", "us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
            "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4), "gflops": round(flops / us / 1e3, 1),
            "tokens_per_s": round(n / us * 1e6, 1), "from_dram": nbytes > 126e6}


def delta_scan(a) -> dict:
    """The gated delta rule's kernel: ``batch`` requests of ``tokens`` tokens each.  One token per request is bound by
    the state it reads and writes; a prompt portion by the walk along its tokens."""
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    inner, ch = a.heads * a.head_dim, a.heads * a.head_dim + 2 * a.key_heads * a.key_dim
    n = a.batch * a.tokens
    qkv = (torch.randn((n, ch), device="cuda") * 0.3).to(dtype)
    proj = torch.randn((n, 2 * a.heads), device="cuda").to(dtype)
    vec = [torch.randn(a.heads, device="cuda") for _ in range(2)]
    state = torch.zeros((a.batch, a.heads, a.head_dim, a.key_dim), device="cuda")
    y = torch.empty((n, inner), device="cuda")
    starts = (torch.arange(a.batch + 1, dtype=torch.int32) * a.tokens).cuda()
    slots = torch.arange(a.batch, dtype=torch.int32).cuda()
    scratch = torch.empty(kernels.delta_scratch_floats(n, a.heads, a.key_heads, a.key_dim, a.head_dim), device="cuda")
    fn = lambda: kernels.delta_scan(qkv, proj, 0, a.heads, vec[0], vec[1], state, a.batch, starts, slots, y, a.key_heads, a.key_dim,  # noqa: E731
                                    scratch)
    us = _time(fn, a.iters, a.warmup)
    item = 2 if dtype == torch.bfloat16 else 4
    nbytes = 2 * state.numel() * 4 + n * (ch * item + inner * 4)
    flops = 8.0 * n * a.heads * a.key_dim * a.head_dim          # two read-outs, the decay and the write, each over the matrix
    return {"case": "delta-scan", "us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
            "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4), "gflops": round(flops / us / 1e3, 1),
            "tokens_per_s": round(n / us * 1e6, 1), "from_dram": nbytes > 126e6}


def routed_experts(a) -> dict:
    """The routed experts' three kernels (router with lists, gate/up product, down product) over ``tokens`` rows, and
    the dense gated feed-forward of equal work per token (``top * ff`` wide) through the library product beside them.
    Few rows are bound by the weights of the chosen experts (every expert's, from about ``experts / top`` rows on),
    many rows by the products' arithmetic."""
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    n, E, top, ff, h = a.tokens, a.experts, a.top, a.ff, a.width
    item = 2 if dtype == torch.bfloat16 else 4
    reps = max(1, int(300e6 // (3 * E * ff * h * item)) + 1)       # rotate over copies of the weights: more than L2 in total
    wgu = [(torch.randn((E, 2 * ff, h), device="cuda") * 0.02).to(dtype) for _ in range(reps)]
    wd = [(torch.randn((E, h, ff), device="cuda") * 0.02).to(dtype) for _ in range(reps)]
    router = torch.randn((E, h), device="cuda") * 0.05
    x = torch.randn((n, h), device="cuda").to(dtype)
    lists = torch.empty(kernels.moe_lists_ints(n, E, top), dtype=torch.int32, device="cuda")
    score = torch.empty(n * top, device="cuda")
    act = torch.empty((n * top, ff), dtype=dtype, device="cuda")
    parts = torch.empty((top, n, h), device="cuda")
    state = {"i": 0}

    def rotate():
        state["i"] = (state["i"] + 1) % reps
        return state["i"]

    tc = kernels.moe_tc_supported(dtype, h, ff) and not getattr(a, "general", False)     # as the feed-forward part chooses
    tile_rows = kernels.moe_tc_tile_rows(n, E, top) if tc else 0
    if getattr(a, "ungated", False):
        return _routed_experts_ungated(a, x, router, wgu, wd, lists, score, act, parts, tc, tile_rows, rotate, reps, item)
    kernels.moe_route(x, router, top, lists, score, tile_rows)
    used = int((lists[2 * n * top: 2 * n * top + E] > 0).sum())     # experts that some row chose
    us_route = _time(lambda: kernels.moe_route(x, router, top, lists, score, tile_rows), a.iters, a.warmup)
    us_gather = 0.0
    if tc:
        xs = torch.empty((n * top, h), dtype=dtype, device="cuda")
        kernels.moe_tc_gather(x, lists, score, E, top, xs)
        us_gather = _time(lambda: kernels.moe_tc_gather(x, lists, score, E, top, xs), a.iters, a.warmup)
        us_up = _time(lambda: kernels.moe_tc_gate_up(xs, wgu[rotate()], lists, top, tile_rows, act), max(a.iters, 2 * reps), a.warmup)
        us_down = _time(lambda: kernels.moe_tc_down(act, wd[rotate()], lists, top, tile_rows, parts), max(a.iters, 2 * reps), a.warmup)
    else:
        us_up = _time(lambda: kernels.moe_gate_up(x, wgu[rotate()], lists, score, top, act), max(a.iters, 2 * reps), a.warmup)
        us_down = _time(lambda: kernels.moe_down(act, wd[rotate()], lists, top, parts), max(a.iters, 2 * reps), a.warmup)
    # the dense feed-forward of the same arithmetic per token
    dgu = [(torch.randn((2 * top * ff, h), device="cuda") * 0.02).to(dtype) for _ in range(max(1, reps // 4))]
    dd = [(torch.randn((h, top * ff), device="cuda") * 0.02).to(dtype) for _ in range(max(1, reps // 4))]
    gu = torch.empty((n, 2 * top * ff), dtype=dtype, device="cuda")
    dact = torch.empty((n, top * ff), dtype=dtype, device="cuda")
    dout = torch.empty((n, h), dtype=dtype, device="cuda")
    us_dense_up = _time(lambda: kernels.linear(x, dgu[rotate() % len(dgu)], gu), a.iters, a.warmup)
    us_dense_down = _time(lambda: kernels.linear(dact, dd[rotate() % len(dd)], dout), a.iters, a.warmup)
    flops_up, flops_down = 4.0 * n * top * ff * h, 2.0 * n * top * ff * h
    bytes_up, bytes_down = used * 2 * ff * h * item + n * h * item + n * top * ff * item, used * ff * h * item + n * top * (ff * item + h * 4)

    def line(us, flops, nbytes):
        return {"us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4),
                "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4)}

    dense_bytes_up, dense_bytes_down = 2 * top * ff * h * item + n * h * item, top * ff * h * item + n * top * ff * item
    return {"case": "routed-experts", "tokens": n, "experts": E, "top": top, "ff": ff, "width": h, "experts_used": used,
            "tensor_cores": bool(tc), "tile_rows": tile_rows, "route_us": round(us_route, 2), "gather_us": round(us_gather, 2), "gate_up": line(us_up, flops_up, bytes_up), "down": line(us_down, flops_down, bytes_down),
            "dense_gate_up": line(us_dense_up, flops_up, dense_bytes_up), "dense_down": line(us_dense_down, flops_down, dense_bytes_down)}


def _routed_experts_ungated(a, x, router, wgu, wd, lists, score, act, parts, tc, tile_rows, rotate, reps, item) -> dict:
    """The same for experts without a gate branch (one up product with the square of relu), softmax scores over groups
    of experts and the weight on the down product's output."""
    n, E, top, ff, h = a.tokens, a.experts, a.top, a.ff, a.width
    groups = tuple(a.groups) if getattr(a, "groups", None) else None
    wu = [w[:, :ff].contiguous() for w in wgu]
    route = lambda: kernels.moe_route(x, router, top, lists, score, tile_rows, scores="softmax", groups=groups)   # noqa: E731
    route()
    used = int((lists[2 * n * top: 2 * n * top + E] > 0).sum())
    us_route = _time(route, a.iters, a.warmup)
    us_gather = 0.0
    if tc:
        xs = torch.empty((n * top, h), dtype=x.dtype, device="cuda")
        kernels.moe_tc_gather(x, lists, None, E, top, xs)
        us_gather = _time(lambda: kernels.moe_tc_gather(x, lists, None, E, top, xs), a.iters, a.warmup)
        us_up = _time(lambda: kernels.moe_tc_up_act(xs, wu[rotate()], lists, top, tile_rows, act), max(a.iters, 2 * reps), a.warmup)
        us_down = _time(lambda: kernels.moe_tc_down(act, wd[rotate()], lists, top, tile_rows, parts, out_score=score),
                        max(a.iters, 2 * reps), a.warmup)
    else:
        us_up = _time(lambda: kernels.moe_up_act(x, wu[rotate()], lists, top, act), max(a.iters, 2 * reps), a.warmup)
        us_down = _time(lambda: kernels.moe_down(act, wd[rotate()], lists, top, parts, out_score=score), max(a.iters, 2 * reps), a.warmup)
    flops = 2.0 * n * top * ff * h
    bytes_up = used * ff * h * item + n * h * item + n * top * ff * item
    bytes_down = used * ff * h * item + n * top * (ff * item + h * 4)

    def line(us, nbytes):
        return {"us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "frac_bf16": round(flops / us / 1e6 / BF16_TFLOPS, 4),
                "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / HBM_GBS, 4)}

    return {"case": "routed-experts", "form": "ungated", "tokens": n, "experts": E, "top": top, "ff": ff, "width": h,
            "experts_used": used, "tensor_cores": bool(tc), "tile_rows": tile_rows, "route_us": round(us_route, 2),
            "gather_us": round(us_gather, 2), "up": line(us_up, bytes_up), "down": line(us_down, bytes_down)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="edgerag_b200.ops.microbench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="case", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--iters", type=int, default=20)
    common.add_argument("--warmup", type=int, default=3)
    common.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    common.add_argument("--peaks", default=None, help="JSON file with hbm_gbs and bf16_tflops to take fractions of")
    att = argparse.ArgumentParser(add_help=False)
    att.add_argument("--heads", type=int, default=32)
    att.add_argument("--kv-heads", type=int, default=32)
    att.add_argument("--head-dim", type=int, default=64)
    att.add_argument("--page", type=int, default=16)
    att.add_argument("--window", type=int, default=0, help="keys a query sees behind itself (0: all)")
    att.add_argument("--keep-first", type=int, default=0, help="with a window: first keys that stay visible")
    att.add_argument("--chunk", type=int, default=0, help="instead of a window: a query sees its own run of this many positions")
    att.add_argument("--sequential-pages", action="store_true", help="pages in order instead of shuffled")
    d = sub.add_parser("decode-attention", parents=[common, att])
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=8192)
    d.add_argument("--split", type=int, default=0, help="keys per split; 0: the engine's choice for this batch")
    d.add_argument("--kernel", choices=["bulk", "gqa", "general"], default="bulk")
    d.add_argument("--head-group", type=int, default=0, help="kv heads per block of the bulk kernel; 0: its own choice")
    d.add_argument("--cold", action="store_true", help="rotate over several caches so that none is found in L2")
    p = sub.add_parser("prefill-attention", parents=[common, att])
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--past", type=int, default=0)
    p.add_argument("--key-splits", type=int, default=0, help="ranges every block's keys are cut into; 0: the engine's choice")
    p.add_argument("--kernel", choices=["tc", "general"], default="tc")
    g = sub.add_parser("linear", parents=[common])
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=6144)
    g.add_argument("--k", type=int, default=2048)
    g.add_argument("--out32", action="store_true")
    g.add_argument("--library", action="store_true", help="force the library product (cuBLASLt) also for few rows")
    g.add_argument("--tc", action="store_true", help="the TMA + tcgen05 weight-streaming kernel (up to 64 rows)")
    g.add_argument("--parts", action="store_true", help="the slices of k as float32 partial results (17 to 64 rows, a weight of few rows)")
    g.add_argument("--glu", action="store_true", help="the gated product: w is [gate; up] of n rows, out has n / 2 columns")
    k = sub.add_parser("step-kernels", parents=[common])
    k.add_argument("--layers", type=int, default=4)
    k.add_argument("--batch", type=int, default=8)
    k.add_argument("--context", type=int, default=8192)
    k.add_argument("--tokens", type=int, default=2048)
    k.add_argument("--heads", type=int, default=32)
    k.add_argument("--kv-heads", type=int, default=32)
    k.add_argument("--config-json", default=None, help="a config.json of any registered architecture instead of the SmolVLM-2.2B sizes")
    k.add_argument("--rows", type=int, default=12, help="kernels listed per table")
    t = sub.add_parser("step-timeline", parents=[common])
    t.add_argument("--layers", type=int, default=4)
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=640)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=32)
    la = sub.add_parser("latent-attention", parents=[common])
    la.add_argument("--heads", type=int, default=16)
    la.add_argument("--rank", type=int, default=512, help="width of the cached latent")
    la.add_argument("--rot", type=int, default=64, help="width of the shared rotated key part")
    la.add_argument("--page", type=int, default=16)
    la.add_argument("--batch", type=int, default=8)
    la.add_argument("--context", type=int, default=8192)
    la.add_argument("--tokens", type=int, default=0, help="prompt tokens (0: single tokens of --batch requests)")
    la.add_argument("--past", type=int, default=0)
    la.add_argument("--split", type=int, default=0)
    la.add_argument("--cold", action="store_true")
    la.add_argument("--kernel", choices=["mma", "general"], default="mma", help="tensor cores (bfloat16) or the general kernel")
    la.add_argument("--window", type=int, default=0, help="keys a query sees behind itself (0: all)")
    da = sub.add_parser("diff-attention", parents=[common])
    da.add_argument("--heads", type=int, default=16)
    da.add_argument("--kv-heads", type=int, default=4)
    da.add_argument("--dim", type=int, default=64, help="entries of one score map of a head")
    da.add_argument("--vdim", type=int, default=128)
    da.add_argument("--page", type=int, default=16)
    da.add_argument("--batch", type=int, default=8)
    da.add_argument("--context", type=int, default=8192)
    da.add_argument("--tokens", type=int, default=0, help="prompt tokens (0: single tokens of --batch requests)")
    da.add_argument("--past", type=int, default=0)
    da.add_argument("--window", type=int, default=1024)
    da.add_argument("--softcap", type=float, default=30.0)
    da.add_argument("--split", type=int, default=0)
    da.add_argument("--cold", action="store_true")
    da.add_argument("--kernel", choices=["mma", "general"], default="mma", help="tensor cores (bfloat16) or the general kernel")
    ss = sub.add_parser("ssm-scan", parents=[common])
    ss.add_argument("--heads", type=int, default=64)
    ss.add_argument("--head-dim", type=int, default=64)
    ss.add_argument("--state", type=int, default=128)
    ss.add_argument("--groups", type=int, default=8)
    ss.add_argument("--batch", type=int, default=8)
    ss.add_argument("--tokens", type=int, default=1)
    ds = sub.add_parser("delta-scan", parents=[common])
    ds.add_argument("--heads", type=int, default=32)
    ds.add_argument("--head-dim", type=int, default=128, help="entries of a value")
    ds.add_argument("--key-heads", type=int, default=16)
    ds.add_argument("--key-dim", type=int, default=128)
    ds.add_argument("--batch", type=int, default=8)
    ds.add_argument("--tokens", type=int, default=1)
    re = sub.add_parser("routed-experts", parents=[common])
    re.add_argument("--tokens", type=int, default=8)
    re.add_argument("--width", type=int, default=2048)
    re.add_argument("--ff", type=int, default=1024)
    re.add_argument("--experts", type=int, default=32)
    re.add_argument("--top", type=int, default=4)
    re.add_argument("--general", action="store_true", help="the products on CUDA cores (what float32 runs) instead of tensor cores")
    re.add_argument("--ungated", action="store_true", help="experts without a gate branch, softmax scores, the weight on the output")
    re.add_argument("--groups", type=int, nargs=2, default=None, help="with --ungated: (count, keep) of the router's groups")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    fn = {"decode-attention": decode_attention, "prefill-attention": prefill_attention, "linear": linear,
          "step-kernels": step_kernels, "step-timeline": step_timeline, "latent-attention": latent_attention,
          "ssm-scan": ssm_scan, "delta-scan": delta_scan, "routed-experts": routed_experts, "diff-attention": diff_attention}[a.case]
    load_peaks(a.peaks)
    result = fn(a)
    result["peaks"] = PEAKS_FROM
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
