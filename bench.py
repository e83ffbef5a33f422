#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  A "step" is one decode step of the batch (default 8 requests, each holding a
2,048-token prompt, context 4,096).  ``value`` is decoded tokens per second over exactly K steps,
timed with CUDA events (``ms_per_step_sd``: the spread of five equal parts of them); ``e2e`` is the same
through ``Engine.step``'s own loop with host token ids in and out; ``prefill`` is a 2,048-token prompt in one
step; ``roofline`` compares the bytes a decode step must read with the measured copy bandwidth; ``points``
holds decode rates at batch 1 and 64 with their fractions of that bandwidth, the end-to-end rate with the command
line's default sampling instead of greedy choice (``e2e_b8_sampled``), the batch-8 rate with the positions
of the published checkpoints (40,960: block tables and descriptions ten times as wide), and the two other
workloads that the baseline names (Qwen3-0.6B shape, 256 requests at once; Qwen3-32B shape, 8 requests of
8,192 tokens in portions of 2,048), each through the engine's own scheduler.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The layer sizes of Qwen3-8B (the reference publishes no number of its own on it: the roofline is the yardstick).
CONFIG_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 4096, "tie_word_embeddings": False, "hidden_act": "silu",
}
FULL_LAYERS = 36
PROMPT_LEN = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, interval_ms=200):
        self.rows, self.proc, self.interval_ms = [], None, interval_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.interval_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, lo=0, hi=None):
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def model_numbers(config: dict) -> dict:
    """Bytes and flops of a model from its configuration (bfloat16 weights and cache)."""
    H, I, L = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    nh, nkv, d, V = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"], config["vocab_size"]
    layer_params = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I
    # what a decode step reads once: every layer's matrices and the head (the embedding table only by a few rows)
    return {"layer_params": layer_params, "weight_bytes": 2 * (L * layer_params + V * H),
            "kv_bytes_per_token": 2 * L * nkv * d * 2, "L": L, "H": H, "I": I, "nh": nh, "nkv": nkv, "d": d, "V": V}


def prefill_flops(m: dict, n_new: int, n_before: int, n_logit_rows: int = 1) -> float:
    """Matrix products of n_new tokens plus causal attention over n_before cached and the new tokens."""
    gemm = 2.0 * n_new * m["L"] * m["layer_params"] + 2.0 * n_logit_rows * m["V"] * m["H"]
    attn = m["L"] * 4.0 * m["nh"] * m["d"] * (n_new * n_before + n_new * (n_new + 1) / 2)
    return gemm + attn


def workload(shape: dict, n_requests: int, prompt_lens, max_tokens: int, tokens_per_step: int, prefill_chunk, pk: dict,
             max_context: int, seed: int = 7) -> dict:
    """Requests through the engine's own scheduler, host token ids in and out: all added at once, prompts cut into
    portions, then decoding.  Times: the wall clock around synchronised sections (the loop is the product's)."""
    import torch

    from inferrs_b200 import SamplingParams
    from inferrs_b200.engine.engine import Engine
    config = dict({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936,
                   "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "hidden_act": "silu",
                   "max_position_embeddings": max_context}, **shape)
    m = model_numbers(config)
    block = 16
    per_request = (max(prompt_lens) + max_tokens + block) // block
    eng = Engine(config=config, random_weights=0, dtype="bf16", block_size=block, num_blocks=n_requests * per_request,
                 max_batch_size=n_requests, max_tokens_per_step=tokens_per_step, prefill_chunk=prefill_chunk)
    eng.warm_up()
    g = torch.Generator().manual_seed(seed)
    sp = SamplingParams.greedy(max_tokens=max_tokens, ignore_eos=True)
    for n in prompt_lens:
        eng.add_request(torch.randint(0, config["vocab_size"], (n,), generator=g).tolist(), sp)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_prompts_in, steps, mixed = None, 0, 0
    while eng.has_work():
        prompts_left = len(eng.scheduler.waiting) + sum(r.n_pending > 1 for r in eng.scheduler.running)
        eng.step()
        steps += 1
        mixed += prompts_left > 0
        if t_prompts_in is None and prompts_left == 0:
            torch.cuda.synchronize()
            t_prompts_in = time.perf_counter()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    st = eng.stats()
    if st["free_pages"] != st["pages"] or st["kernel_errors"]:
        raise RuntimeError(f"the workload left pages behind or a kernel reported an error: {st}")
    n_prompt, n_gen = sum(prompt_lens), n_requests * max_tokens
    out = {"tok_s": round((n_prompt + n_gen) / (t1 - t0), 1), "s": round(t1 - t0, 3), "steps": steps}
    if t_prompts_in is not None and steps > mixed + 1:
        t_in, t_dec = t_prompts_in - t0, t1 - t_prompts_in
        n_dec_steps = steps - mixed - 1
        # prompts: every prompt's products and its causal attention, against the bf16 peak that is sustained
        flops = sum(prefill_flops(m, n, 0) for n in prompt_lens)
        peak = (pk.get("bf16_tflops_sustained") or pk["bf16_tflops"]) * 1e12
        out.update({"prefill_tok_s": round(n_prompt / t_in, 1), "prefill_frac": round(flops / t_in / peak, 4),
                    "decode_tok_s": round(n_requests * n_dec_steps / t_dec, 1)})
        # decode: weights once per step plus the live requests' cache at the mean length of the decode phase
        mean_ctx = sum(prompt_lens) / n_requests + max_tokens / 2
        step_bytes = m["weight_bytes"] + n_requests * mean_ctx * m["kv_bytes_per_token"]
        out["decode_frac"] = round(step_bytes / (t_dec / n_dec_steps) / 1e9 / pk["hbm_gbs"], 4)
    del eng
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has, for quick runs")
    ap.add_argument("--clock-interval-ms", type=int, default=200, help="how often nvidia-smi is asked for the clocks")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points and the prefill")
    ap.add_argument("--no-workloads", action="store_true", help="skip the Qwen3-0.6B and Qwen3-32B workloads")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace (cargo/rustc absent, "
                          "no network for crates): it cannot be installed or run here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import gc

    import torch

    from inferrs_b200 import SamplingParams, kernels
    from inferrs_b200.engine.batch import StepEntry
    from inferrs_b200.engine.engine import Engine

    torch.cuda.set_device(0)
    pk = peaks()
    config = dict(CONFIG_8B, num_hidden_layers=args.layers)
    block = 16
    biggest = max(args.batch, 1 if args.no_points else 64)
    ctx_pages = CONFIG_8B["max_position_embeddings"] // block
    eng = Engine(config=config, random_weights=0, dtype="bf16", block_size=block, num_blocks=biggest * ctx_pages,
                 max_batch_size=biggest, max_tokens_per_step=8192)
    vocab = config["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    m = model_numbers(config)
    L, H, I, nh, nkv, d = m["L"], m["H"], m["I"], m["nh"], m["nkv"], m["d"]

    def prompt():
        return torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()

    def decode_steps(runner, batch: int, steps: int, warmup: int, parts: int = 5):
        """(ms per step, its spread over `parts` equal parts of the steps, launches per step): `batch` requests with
        PROMPT_LEN tokens cached, then exactly `steps` timed decode steps."""
        rids = [("b", batch, i) for i in range(batch)]
        for i in range(0, batch, 4):  # prompts go in four at a time
            chunk = rids[i:i + 4]
            for r in chunk:
                runner.admit(r)
            runner.step([StepEntry(r, prompt(), []) for r in chunk])
        toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        out = torch.empty((batch,), dtype=torch.int32, device="cuda")

        def one():
            logits = runner.step([StepEntry(r, [t], [0]) for r, t in zip(rids, toks)], own_output=False)
            kernels.argmax(logits, out, torch.bfloat16)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        n0 = kernels.launch_count()
        parts = max(1, min(parts, steps))
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(parts + 1)]
        edges = [round(k * steps / parts) for k in range(parts + 1)]
        marks[0].record()
        for k in range(parts):
            for _ in range(edges[k + 1] - edges[k]):
                one()
            marks[k + 1].record()
        torch.cuda.synchronize()
        launches = (kernels.launch_count() - n0) / steps
        for r in rids:
            runner.release(r)
        per_part = [marks[k].elapsed_time(marks[k + 1]) / (edges[k + 1] - edges[k]) for k in range(parts)]
        sd = statistics.stdev(per_part) if parts > 1 else 0.0
        return marks[0].elapsed_time(marks[-1]) / steps, sd, launches

    def hbm_frac(batch, ms, ctx_mid):
        return (m["weight_bytes"] + batch * ctx_mid * m["kv_bytes_per_token"]) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

    clocks = ClockSampler(args.clock_interval_ms)
    clocks.start()
    time.sleep(0.3)
    lo = clocks.mark()
    ms, ms_sd, launches = decode_steps(eng.runner, args.batch, args.steps, args.warmup)
    hi = clocks.mark()
    value = args.batch * 1e3 / ms
    ctx_mid = PROMPT_LEN + args.warmup + args.steps / 2
    frac = hbm_frac(args.batch, ms, ctx_mid)

    # end to end: the engine's own loop, host token ids in, host token ids out, every step
    def end_to_end(sp):
        for _ in range(args.batch):
            eng.add_request(prompt(), sp)
        reqs = list(eng.scheduler.waiting)
        while any(not r.output for r in reqs):
            eng.step()
        for _ in range(args.warmup):
            eng.step()
        torch.cuda.synchronize()
        parts_ms, n_done = [], 0
        n_loop = args.steps - 1
        edges = [round(k * n_loop / 5) for k in range(6)]
        t0 = time.perf_counter()
        for k in range(5):
            tk = time.perf_counter()
            done = 0
            for _ in range(edges[k + 1] - edges[k]):
                if not eng.has_work():
                    break
                eng.step()
                done += 1
            torch.cuda.synchronize()
            if done:
                parts_ms.append((time.perf_counter() - tk) * 1e3 / done)
            n_done += done
        ms_step = (time.perf_counter() - t0) * 1e3 / max(n_done, 1)
        while eng.has_work():
            eng.step()
        return ms_step, parts_ms

    n_new = args.steps + args.warmup + 16          # no request ends inside the timed loop
    e2e_ms, e2e_parts = end_to_end(SamplingParams.greedy(max_tokens=n_new, ignore_eos=True))
    # the step's description as it is copied from pinned host memory: the replayed graph's whole fixed buffer
    graphs = eng.runner.graphs
    meta_ints = graphs.captured[graphs.bucket_for(args.batch)].buffer.numel() if graphs is not None else 0

    out = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, 2,048-token prompts cached, 1xB200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_sd": round(ms_sd, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_full": FULL_LAYERS, "hidden": H, "heads": nh,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": vocab, "global_batch": args.batch,
                   "seq_len": CONFIG_8B["max_position_embeddings"], "prompt_len": PROMPT_LEN, "block_size": block,
                   "parallelism": "none", "l2": "inputs larger than L2 (weights read once per step)",
                   "sampling": "greedy"},
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "ms_per_step_sd": round(statistics.stdev(e2e_parts), 4) if len(e2e_parts) > 1 else 0.0,
                "h2d_bytes_per_step": 4 * meta_ints, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(round(launches * args.steps)),
        "roofline": {"bound": "hbm", "achieved": round(frac * pk["hbm_gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(frac, 4), "of": pk["source"]},
        "clocks": clocks.summary(lo, hi),
    }

    if not args.no_points:
        # the same loop with the sampling that the command line starts with (temperature 0.7, top-k 50, top-p 0.9,
        # repetition penalty 1.1 over the last 64 tokens)
        sampled_ms, _ = end_to_end(SamplingParams(max_tokens=n_new, ignore_eos=True, seed=1))
        # prefill: one 2,048-token prompt in one step
        runner = eng.runner
        times = []
        for i in range(7):
            rid = ("p", i)
            runner.admit(rid)
            p = prompt()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step([StepEntry(rid, p, [PROMPT_LEN - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.release(rid)
            if i >= 2:
                times.append(a.elapsed_time(b))
        pms = statistics.median(times)
        flops = prefill_flops(m, PROMPT_LEN, 0)
        out["prefill"] = {"value": round(PROMPT_LEN * 1e3 / pms, 1), "tokens": PROMPT_LEN, "ms": round(pms, 3),
                          "ms_sd": round(statistics.stdev(times), 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "tflops": round(flops / (pms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
                          "of": pk["source"]}
        if pk.get("bf16_tflops_sustained"):
            # the same library product back to back for seconds, under the power cap: what a step of tens of
            # milliseconds can be compared with; "frac" stays the fraction of the burst figure
            out["prefill"]["frac_of_sustained"] = round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        points = {}
        for b in (1, 64):
            n_b = 64 if b == 64 else 128
            ms_b, sd_b, _ = decode_steps(runner, b, n_b, 4)
            points[f"decode_b{b}"] = round(b * 1e3 / ms_b, 1)
            points[f"decode_b{b}_ms_sd"] = round(sd_b, 4)
            points[f"decode_b{b}_frac"] = round(hbm_frac(b, ms_b, PROMPT_LEN + 4 + n_b / 2), 4)
        points[f"e2e_b{args.batch}_sampled"] = round(args.batch * 1e3 / sampled_ms, 1)
        out["points"] = points
    del eng
    gc.collect()
    torch.cuda.empty_cache()

    if not args.no_points:
        # the positions of the published checkpoints (40,960): rotation tables, block tables of replayed steps and
        # their descriptions are ten times as wide; same requests, same step otherwise
        wide = dict(config, max_position_embeddings=40960)
        eng = Engine(config=wide, random_weights=0, dtype="bf16", block_size=block, num_blocks=40960 // block + args.batch * ctx_pages,
                     max_batch_size=args.batch, max_tokens_per_step=8192)
        ms_w, sd_w, _ = decode_steps(eng.runner, args.batch, 64, 4)
        out["points"][f"decode_b{args.batch}_pos40960"] = round(args.batch * 1e3 / ms_w, 1)
        out["points"][f"decode_b{args.batch}_pos40960_frac"] = round(hbm_frac(args.batch, ms_w, PROMPT_LEN + 4 + 32), 4)
        del eng
        gc.collect()
        torch.cuda.empty_cache()

    if not args.no_workloads and not args.no_points and args.layers == FULL_LAYERS:
        from inferrs_b200.microbench import SHAPES
        g = torch.Generator().manual_seed(7)
        lens = torch.randint(16, 1025, (256,), generator=g).tolist()
        w = workload(SHAPES["0.6b"], 256, lens, 128, 2048, 2048, pk, max_context=4096)
        out["points"].update({f"wl_06b_{k}": v for k, v in w.items()})
        w = workload(SHAPES["32b"], 8, [8192] * 8, 128, 2048, 2048, pk, max_context=8448)
        out["points"].update({f"wl_32b_{k}": v for k, v in w.items()})
    clocks.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
