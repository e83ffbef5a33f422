"""Timing of single kernels at given sizes: the commands behind the summaries in ``profiles/``.

    python -m inferrs_b200.microbench gemm --impl tcgen05 --m 8 --n 6144 --k 4096
    python -m inferrs_b200.microbench attention --form decode --batch 8 --context 2048
    python -m inferrs_b200.microbench attention --form prefill --tokens 2048
    python -m inferrs_b200.microbench chain --impl library --m 8 --layers 8
    python -m inferrs_b200.microbench step --form decode --batch 8 --context 2048 --layers 8
    python -m inferrs_b200.microbench step --form decode --batch 8 --context 2048 --layers 3 --trace
    python -m inferrs_b200.microbench workload --shape 0.6b --requests 256 --prompt-min 16 --prompt-max 1024
    python -m inferrs_b200.microbench workload --shape 32b --requests 8 --prompt-min 8192 --prompt-max 8192 \
        --max-context 16384
    python -m inferrs_b200.microbench workload --shape 0.6b --requests 256 --profile-steps 4 --skip-steps 10
    python -m inferrs_b200.microbench sample --rows 8 --top-k 50 --top-p 0.9

Every case is timed with CUDA events after warm-up; between timed launches a buffer larger than the
L2 cache is written, so each launch starts cold.  One JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from . import kernels


def _time(fn, iters: int, flush: bool = True) -> float:
    """Median microseconds of one call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    scrub = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def gemm(args) -> dict:
    if args.impl == "gated":
        # n counts the rows of the stacked gate and up matrices: the output has n / 2 columns
        inner = args.n // 2
        x = torch.randn(args.m, args.k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(2 * inner, args.k, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(args.m, inner, dtype=torch.bfloat16, device="cuda")
        us = _time(lambda: kernels.gemm_swiglu_tcgen05(x, w, out), args.iters)
        gu = x.float() @ w.float().t()
        g, u = gu[:, :inner].bfloat16().float(), gu[:, inner:].bfloat16().float()
        ref = g / (1.0 + torch.exp(-g)) * u
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        byts = 2 * (2 * inner * args.k + args.m * args.k + args.m * inner)
        return {"kernel": "gemm/gated", "m": args.m, "n": 2 * inner, "k": args.k, "us": round(us, 2),
                "GBps": round(byts / us / 1e3, 1), "TFLOPs": round(4 * args.m * inner * args.k / us / 1e6, 1),
                "rel_err": err}
    x = torch.randn(args.m, args.k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(args.n, args.k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(args.m, args.n, dtype=torch.bfloat16, device="cuda")
    fn = {"library": lambda: kernels.gemm_tn_bf16(x, w, out),
          "tcgen05": lambda: kernels.gemm_tn_tcgen05(x, w, out, args.split_k)}[args.impl]
    us = _time(fn, args.iters)
    ref = x.float() @ w.float().t()
    err = float((out.float() - ref).abs().max() / ref.abs().max())
    byts = 2 * (args.n * args.k + args.m * args.k + args.m * args.n)
    flops = 2 * args.m * args.n * args.k
    return {"kernel": f"gemm/{args.impl}", "m": args.m, "n": args.n, "k": args.k, "us": round(us, 2),
            "GBps": round(byts / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1), "rel_err": err}


def attention(args) -> dict:
    nh, nkv, d, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    dev = torch.device("cuda")
    if args.form == "decode":
        lens, new = [args.context] * args.batch, [1] * args.batch
    else:
        lens, new = [args.context_before + args.tokens], [args.tokens]
    pages_per = [(n + ps - 1) // ps for n in lens]
    n_pages = sum(pages_per)
    table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).to(torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = perm[at:at + n]
        at += n
    positions = torch.tensor([p for n, t in zip(lens, new) for p in range(n - t, n)], dtype=torch.int32, device=dev)
    row_request = torch.tensor([r for r, t in enumerate(new) for _ in range(t)], dtype=torch.int32, device=dev)
    q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev)
    n = sum(new)
    q = torch.randn(n, nh, d, device=dev).to(torch.bfloat16)
    k_pages = torch.randn(n_pages, nkv, ps, d, device=dev).to(torch.bfloat16)
    v_pages = torch.randn(n_pages, nkv, ps, d, device=dev).to(torch.bfloat16)
    out = torch.empty(n, nh * d, dtype=torch.bfloat16, device=dev)
    table = table.to(dev)
    scale = d ** -0.5
    if args.form == "decode":
        if args.impl == "mma":
            splits = args.splits or kernels.decode_splits(args.batch, nkv, args.context)
            fn = lambda: kernels.paged_attention_mma(q, k_pages, v_pages, table, row_request, q_start, n, q_start,  # noqa: E731
                                                     positions, scale, None, out, True, splits)
        else:
            splits, min_tiles = kernels.decode_slices(args.batch, nkv, args.max_context or args.context)
            splits, min_tiles = args.splits or splits, args.min_tiles or min_tiles
            fn = lambda: kernels.paged_attention_decode(q, k_pages, v_pages, table, positions, scale, None, out,  # noqa: E731
                                                        splits, min_tiles=min_tiles)
        byts = 2 * 2 * sum(lens) * nkv * d
        flops = 4 * nh * d * sum(lens)
        extra = {"batch": args.batch, "context": args.context, "splits": splits}
    else:
        tpt = kernels.pair_tile_tokens(nh, nkv) if args.impl == "tcgen05-pair" else \
            (kernels.TC_ROWS if args.impl == "tcgen05" else kernels.MMA_KEYS) // (nh // nkv)
        req = [0] * ((args.tokens + tpt - 1) // tpt)
        row0 = list(range(0, args.tokens, tpt))
        tile_req = torch.tensor(req, dtype=torch.int32, device=dev)
        tile_row0 = torch.tensor(row0, dtype=torch.int32, device=dev)
        if args.impl == "tcgen05":
            fn = lambda: kernels.paged_attention_tcgen05(q, k_pages, v_pages, table, tile_req, tile_row0, len(req),  # noqa: E731
                                                         q_start, positions, scale, None, out)
        elif args.impl == "tcgen05-pair":
            fn = lambda: kernels.paged_attention_pair_tcgen05(q, k_pages, v_pages, table, tile_req, tile_row0, len(req),  # noqa: E731
                                                              q_start, positions, scale, None, out)
        else:
            fn = lambda: kernels.paged_attention_mma(q, k_pages, v_pages, table, tile_req, tile_row0, len(req),  # noqa: E731
                                                     q_start, positions, scale, None, out, False)
        byts = 2 * 2 * lens[0] * nkv * d + 2 * 2 * n * nh * d
        t, c = args.tokens, args.context_before
        flops = 4 * nh * d * (t * c + t * (t + 1) // 2)
        extra = {"tokens": args.tokens, "context_before": args.context_before}
    us = _time(fn, args.iters)
    return dict({"kernel": f"attention/{args.form}" + (f"/{args.impl}" if args.form == "prefill" else ""), "heads": nh, "kv_heads": nkv, "head_dim": d, "us": round(us, 2),
                 "GBps": round(byts / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1)}, **extra)


def chain(args) -> dict:
    """The four projections of `layers` decoder layers back to back in one CUDA graph, every layer with weights
    of its own: what a decode step pays for its matrix products, launch gaps and cold starts included."""
    h, inner, qkv = args.hidden, args.inner, args.qkv
    shapes = [(qkv, h), (h, args.attn_out), (2 * inner, h), (h, inner)]
    ws = [[(torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16) for n, k in shapes] for _ in range(args.layers)]
    xs = [torch.randn(args.m, k, device="cuda").to(torch.bfloat16) for _, k in shapes]
    outs = [torch.empty(args.m, n, dtype=torch.bfloat16, device="cuda") for n, _ in shapes]
    if args.impl in ("folded", "persistent"):
        # the products as a decode step has them, norms folded in: o projection into the stream, gate and up with
        # the gate, down into the stream, q/k/v; one kernel each, or all four as one persistent kernel
        res = torch.randn(args.m, h, device="cuda")
        norm = [torch.ones(h, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        act = torch.empty(args.m, inner, dtype=torch.bfloat16, device="cuda")
        bf = torch.bfloat16

        def run():
            for w_qkv, w_o, w_gu, w_d in ws:
                c = kernels.ProductChain() if args.impl == "persistent" else None
                lin = c.linear if c else (lambda x, w, o, sink=None: kernels.linear(x, w, o, bf, sink=sink))
                gated = c.gated_linear if c else (lambda x, w, o: kernels.gated_linear(x, w, o, bf))
                s1 = lin(xs[1], w_o, outs[1], sink=kernels.ResidualSink(res, norm[0], 1e-6))
                gated(s1, w_gu, act)
                s2 = lin(act, w_d, outs[3], sink=kernels.ResidualSink(res, norm[1], 1e-6))
                lin(s2, w_qkv, outs[0])
                if c:
                    c.launch()
    else:
        fn = {"library": kernels.gemm_tn_bf16, "tcgen05": lambda x, w, o: kernels.gemm_tn_tcgen05(x, w, o, 0)}[args.impl]

        def run():
            for layer in ws:
                for x, w, o in zip(xs, layer, outs):
                    fn(x, w, o)

    if args.pdl:
        kernels.gemm_tcgen05_set_pdl(True)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    us = _time(g.replay, args.iters, flush=False) / args.layers
    byts = 2 * sum(n * k for n, k in shapes)
    return {"kernel": f"gemm-chain/{args.impl}", "m": args.m, "layers": args.layers, "us_per_layer": round(us, 2),
            "GBps": round(byts / us / 1e3, 1)}


def _trace(fn, args) -> dict:
    """When every kernel of one step started and ended on the device (CUPTI activity records through
    torch.profiler): kernels that were launched early show their overlap with the kernels before them.
    Times under the profiler are a little longer than without it: read the shares."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        fn()
        fn()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    ev = ev[len(ev) // 2:]                      # the second of the two steps
    t0 = ev[0].time_range.start
    print(f"{'start us':>9} {'end us':>9} {'after the kernel before':>24}  kernel")
    prev_end = None
    for e in ev:
        a, b = e.time_range.start - t0, e.time_range.end - t0
        step_us = "" if prev_end is None else f"{b - prev_end:8.2f}"
        print(f"{a:9.2f} {b:9.2f} {step_us:>24}  {e.name[:60]}")
        prev_end = b if prev_end is None else max(prev_end, b)
    return {"kernel": f"step/{args.form} trace", "batch": args.batch, "context": args.context, "tokens": args.tokens,
            "layers": args.layers, "kernels": len(ev), "us_first_start_to_last_end": round(prev_end, 1)}


def step(args) -> dict:
    """A whole step of a random model with Qwen3-8B layer sizes (fewer layers, so that it is quick): the
    time per layer of a decode step at a batch size and context length, or of one prompt portion."""
    from .engine.batch import StepEntry
    from .engine.loading import random_model
    from .engine.runner import ModelRunner
    from .runtime import Runtime
    config = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": args.layers,
              "hidden_size": args.hidden, "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads,
              "head_dim": args.head_dim, "intermediate_size": args.inner, "vocab_size": args.vocab,
              "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": args.max_context,
              "tie_word_embeddings": False, "hidden_act": "silu"}
    rt = Runtime.cuda(torch.bfloat16)
    spec, weights, _ = random_model(config, 0, rt)
    ps = args.page_size
    n_req = args.batch if args.form == "decode" else 1
    per_req = (args.max_context + ps - 1) // ps
    runner = ModelRunner(spec, weights, rt, page_size=ps, n_pages=n_req * per_req, max_requests=n_req,
                         max_context=args.max_context)
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, args.vocab, (n,), generator=g).tolist()  # noqa: E731
    h, inner, nh, nkv, d = args.hidden, args.inner, args.heads, args.kv_heads, args.head_dim
    layer_params = (nh + 2 * nkv) * d * h + nh * d * h + 3 * h * inner
    if args.form == "decode":
        rids = list(range(args.batch))
        for i in range(0, args.batch, 4):
            for r in rids[i:i + 4]:
                runner.admit(r)
            runner.step([StepEntry(r, toks(args.context), []) for r in rids[i:i + 4]])
        one = toks(args.batch)
        n_steps = min(args.iters, args.max_context - args.context - 4)
        for _ in range(3):
            runner.step([StepEntry(r, [t], [0]) for r, t in zip(rids, one)], own_output=False)
        torch.cuda.synchronize()
        if args.trace:
            return _trace(lambda: runner.step([StepEntry(r, [t], [0]) for r, t in zip(rids, one)], own_output=False),
                          args)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_steps):
            runner.step([StepEntry(r, [t], [0]) for r, t in zip(rids, one)], own_output=False)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / n_steps
        head_bytes = 2 * args.vocab * h
        byts = 2 * args.layers * layer_params + head_bytes + args.batch * args.context * 2 * args.layers * nkv * d * 2
        return {"kernel": "step/decode", "batch": args.batch, "context": args.context, "layers": args.layers,
                "us_per_step": round(us, 1), "us_per_layer": round((us - head_bytes / 6.3e6) / args.layers, 2),
                "tokens_per_s_at_36_layers": round(args.batch * 1e6 / ((us - head_bytes / 6.3e6) / args.layers * 36
                                                                       + head_bytes / 6.3e6), 1),
                "GBps": round(byts / us / 1e3, 1), "note": "per layer: the step less the head product at 6.3 TB/s"}
    if args.trace:
        state = {"i": 1000}

        def one_prompt():
            i = state["i"]
            state["i"] += 1
            runner.admit(i)
            if args.context_before:
                runner.step([StepEntry(i, toks(args.context_before), [])])
            runner.step([StepEntry(i, toks(args.tokens), [args.tokens - 1])])
            runner.release(i)
        for _ in range(3):
            one_prompt()
        return _trace(one_prompt, args)
    times = []
    for i in range(args.iters + 2):
        runner.admit(i)
        if args.context_before:
            runner.step([StepEntry(i, toks(args.context_before), [])])
        p = toks(args.tokens)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry(i, p, [args.tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.release(i)
        if i >= 2:
            times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    us = times[len(times) // 2]
    t, c = args.tokens, args.context_before
    flops = args.layers * (2 * t * layer_params + 4 * nh * d * (t * c + t * (t + 1) // 2)) + 2 * args.vocab * h
    return {"kernel": "step/prefill", "tokens": t, "context_before": c, "layers": args.layers,
            "us_per_step": round(us, 1), "us_per_layer": round(us / args.layers, 1),
            "TFLOPs": round(flops / us / 1e6, 1)}


SHAPES = {
    # layer sizes of the published Qwen3 checkpoints (random weights are made on the device)
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 intermediate_size=3072, tie_word_embeddings=True),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, tie_word_embeddings=False),
    "14b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17408, tie_word_embeddings=False),   # five query heads per key/value head
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, tie_word_embeddings=False),
}


def workload(args) -> dict:
    """Requests through the engine's own scheduler, host token ids in and out, timed by the wall clock:
    ``--requests`` prompts with lengths uniform in [--prompt-min, --prompt-max], ``--max-tokens`` greedy (or, with
    ``--sampled``, sampled) tokens each, all added at once (continuous batching with prompts cut into portions of ``--prefill-chunk``)."""
    import time

    from .engine.engine import Engine
    from .sampling.params import SamplingParams
    config = dict({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": args.vocab,
                   "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "hidden_act": "silu",
                   "max_position_embeddings": args.max_context}, **SHAPES[args.shape])
    if args.layers:
        config["num_hidden_layers"] = args.layers
    per_request = (args.prompt_max + args.max_tokens + args.page_size) // args.page_size
    eng = Engine(config=config, random_weights=0, dtype="bf16", block_size=args.page_size,
                 num_blocks=max(per_request, int(args.requests * per_request * args.cache_share)),
                 max_batch_size=args.requests,
                 max_tokens_per_step=args.tokens_per_step, prefill_chunk=args.prefill_chunk)
    eng.warm_up()
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(args.prompt_min, args.prompt_max + 1, (args.requests,), generator=g).tolist()
    sp = SamplingParams(max_tokens=args.max_tokens, ignore_eos=True, seed=1) if args.sampled \
        else SamplingParams.greedy(max_tokens=args.max_tokens, ignore_eos=True)
    for n in lens:
        eng.add_request(torch.randint(0, args.vocab, (n,), generator=g).tolist(), sp)
    torch.cuda.synchronize()
    if args.profile_steps:
        return _profile_steps(eng, args)
    t0 = time.perf_counter()
    first_decode = None
    steps = mixed = 0
    while eng.has_work():
        waiting_before = len(eng.scheduler.waiting) + sum(r.n_pending > 1 for r in eng.scheduler.running)
        eng.step()
        steps += 1
        mixed += waiting_before > 0
        if first_decode is None and waiting_before == 0:
            torch.cuda.synchronize()
            first_decode = time.perf_counter()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    st = eng.stats()
    eng.runner.manager.check_invariants()
    if st["free_pages"] != st["pages"]:
        raise RuntimeError(f"pages were not given back: {st}")
    out = {"kernel": "workload", "shape": args.shape, "layers": config["num_hidden_layers"], "requests": args.requests,
           "prompt_tokens": sum(lens), "generated_tokens": args.requests * args.max_tokens, "steps": steps,
           "steps_with_prompt_portions": mixed, "preemptions": st["preemptions"], "seconds": round(t1 - t0, 3),
           "generated_tokens_per_s": round(args.requests * args.max_tokens / (t1 - t0), 1),
           "all_tokens_per_s": round((sum(lens) + args.requests * args.max_tokens) / (t1 - t0), 1)}
    if first_decode is not None:
        out["until_all_prompts_are_in_s"] = round(first_decode - t0, 3)
        out["prompt_tokens_per_s_until_then"] = round(sum(lens) / (first_decode - t0), 1)
        out["decode_tokens_per_s_after"] = round(args.requests * (steps - mixed - 1) / max(t1 - first_decode, 1e-9), 1)
    return out


def _profile_steps(eng, args) -> dict:
    """``--skip-steps`` steps of the workload unrecorded, then ``--profile-steps`` steps under the profiler: per kernel how
    far it moved the end of the step on the device ("adds": kernels started early under programmatic dependent launch
    overlap, so their own durations would count time twice) and how often it ran.  Times under the profiler are a few
    percent longer than without it."""
    from torch.profiler import ProfilerActivity, profile
    kinds = []
    for _ in range(args.skip_steps):
        if eng.has_work():
            eng.step()
    torch.cuda.synchronize()
    n = 0
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        while n < args.profile_steps and eng.has_work():
            waiting = len(eng.scheduler.waiting) + sum(r.n_pending > 1 for r in eng.scheduler.running)
            kinds.append("portions" if waiting else "decode")
            eng.step()
            n += 1
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    adds, count, end = {}, {}, None
    for e in events:
        st, en = e.time_range.start, e.time_range.end
        add = en - st if end is None else (en - max(end, st) if en > end else 0.0)
        gap = 0.0 if end is None else max(0.0, st - end)
        end = en if end is None else max(end, en)
        name = e.name.split("(")[0][:64]
        adds[name] = adds.get(name, 0.0) + add
        count[name] = count.get(name, 0) + 1
        key = "(idle between kernels)" if gap < 200.0 else "(idle between steps)"
        adds[key] = adds.get(key, 0.0) + gap
    top = sorted(adds.items(), key=lambda kv: -kv[1])[:14]
    while eng.has_work():       # let the requests end, so that the engine's books close
        eng.step()
    return {"kernel": "workload steps", "shape": args.shape, "steps": n, "with_prompt_portions": kinds.count("portions"),
            "us_per_step": round(sum(adds.values()) / max(n, 1), 1),
            "adds_us_per_step": {k: [round(v / max(n, 1), 1), round(count.get(k, 0) / max(n, 1), 1)] for k, v in top}}


def sample(args) -> dict:
    """The selection kernel alone: one token per row of float32 logits [rows, vocab]."""
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn((args.rows, args.vocab), device=dev, generator=g) * 3.0
    t = torch.full((args.rows,), args.temperature, device=dev)
    tk = torch.full((args.rows,), args.top_k, dtype=torch.int32, device=dev)
    tp = torch.full((args.rows,), args.top_p, device=dev)
    mp = torch.full((args.rows,), args.min_p, device=dev)
    u = torch.rand((args.rows,), device=dev, generator=g)
    out = torch.empty((args.rows,), dtype=torch.int32, device=dev)
    us = _time(lambda: kernels.sample(logits, t, tk, tp, mp, u, out, torch.bfloat16, cluster=args.cluster), args.iters)
    return {"kernel": "sample", "rows": args.rows, "vocab": args.vocab, "temperature": args.temperature,
            "top_k": args.top_k, "top_p": args.top_p, "min_p": args.min_p, "cluster": args.cluster, "us": round(us, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inferrs_b200.microbench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--full-tiles", action="store_true",
                    help="tcgen05 products keep every tile at the MMA's height instead of spreading their rows "
                         "evenly over the SMs")
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--impl", choices=["library", "tcgen05", "gated"], default="tcgen05",
                   help="gated: both products of a gated feed-forward and the gate in one tcgen05 kernel")
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=6144)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--split-k", type=int, default=0)
    g.add_argument("--iters", type=int, default=20)
    g.set_defaults(fn=gemm)
    a = sub.add_parser("attention")
    a.add_argument("--form", choices=["decode", "prefill"], default="decode")
    a.add_argument("--impl", choices=["mma", "tcgen05", "tcgen05-pair"], default="tcgen05", help="which kernel (decode form: mma = cp.async kernel, tcgen05 = TMA-fed kernel)")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--context", type=int, default=2048)
    a.add_argument("--tokens", type=int, default=2048)
    a.add_argument("--context-before", type=int, default=0)
    a.add_argument("--splits", type=int, default=0)
    a.add_argument("--min-tiles", type=int, default=0, help="decode form: fewest 64-key tiles per slice (0: as the engine chooses)")
    a.add_argument("--max-context", type=int, default=0, help="decode form: the context that the grid is sized for")
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--iters", type=int, default=20)
    a.set_defaults(fn=attention)
    c = sub.add_parser("chain")
    c.add_argument("--impl", choices=["library", "tcgen05", "folded", "persistent"], default="library",
                   help="folded: the products with the norms folded in, one kernel each; persistent: the same four as one kernel")
    c.add_argument("--m", type=int, default=8)
    c.add_argument("--layers", type=int, default=8)
    c.add_argument("--hidden", type=int, default=4096)
    c.add_argument("--inner", type=int, default=12288)
    c.add_argument("--qkv", type=int, default=6144)
    c.add_argument("--attn-out", type=int, default=4096)
    c.add_argument("--iters", type=int, default=10)
    c.add_argument("--pdl", action="store_true", help="programmatic dependent launch between the kernels (not for the library's)")
    c.set_defaults(fn=chain)
    st = sub.add_parser("step")
    st.add_argument("--form", choices=["decode", "prefill"], default="decode")
    st.add_argument("--batch", type=int, default=8)
    st.add_argument("--context", type=int, default=2048)
    st.add_argument("--tokens", type=int, default=2048)
    st.add_argument("--context-before", type=int, default=0)
    st.add_argument("--max-context", type=int, default=4096)
    st.add_argument("--layers", type=int, default=8)
    st.add_argument("--hidden", type=int, default=4096)
    st.add_argument("--inner", type=int, default=12288)
    st.add_argument("--heads", type=int, default=32)
    st.add_argument("--kv-heads", type=int, default=8)
    st.add_argument("--head-dim", type=int, default=128)
    st.add_argument("--vocab", type=int, default=151936)
    st.add_argument("--page-size", type=int, default=16)
    st.add_argument("--iters", type=int, default=64)
    st.add_argument("--trace", action="store_true", help="print when every kernel of one step started and ended")
    st.set_defaults(fn=step)
    sm = sub.add_parser("sample")
    sm.add_argument("--rows", type=int, default=8)
    sm.add_argument("--vocab", type=int, default=151936)
    sm.add_argument("--temperature", type=float, default=0.7)
    sm.add_argument("--top-k", type=int, default=50)
    sm.add_argument("--top-p", type=float, default=0.9)
    sm.add_argument("--min-p", type=float, default=0.0)
    sm.add_argument("--cluster", type=int, default=0, help="CTAs per row (1, 2, 4, 8); 0 lets the library choose")
    sm.add_argument("--iters", type=int, default=20)
    sm.set_defaults(fn=sample)

    wl = sub.add_parser("workload")
    wl.add_argument("--shape", choices=sorted(SHAPES), default="0.6b")
    wl.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has, for quick runs")
    wl.add_argument("--requests", type=int, default=256)
    wl.add_argument("--prompt-min", type=int, default=16)
    wl.add_argument("--prompt-max", type=int, default=1024)
    wl.add_argument("--max-tokens", type=int, default=128)
    wl.add_argument("--tokens-per-step", type=int, default=2048)
    wl.add_argument("--prefill-chunk", type=int, default=2048)
    wl.add_argument("--max-context", type=int, default=4096)
    wl.add_argument("--vocab", type=int, default=151936)
    wl.add_argument("--page-size", type=int, default=16)
    wl.add_argument("--cache-share", type=float, default=1.0,
                    help="pages as a share of what all requests need at once (less: requests are preempted)")
    wl.add_argument("--sampled", action="store_true",
                    help="the command line's default sampling (temperature 0.7, top-k 50, top-p 0.9, repetition "
                         "penalty 1.1) instead of greedy choice")
    wl.add_argument("--profile-steps", type=int, default=0,
                    help="instead of timing the workload: record this many steps and print what every kernel adds")
    wl.add_argument("--skip-steps", type=int, default=10, help="... after this many unrecorded steps")
    wl.set_defaults(fn=workload)
    args = ap.parse_args(argv)
    if args.full_tiles:
        kernels.gemm_tcgen05_set_even_tiles(False)
    print(json.dumps(args.fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
