#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  A "step" is one decode step of the batch (default 8 requests, each holding a
2,048-token prompt, context 4,096).  ``value`` is decoded tokens per second over exactly K steps,
timed with CUDA events; ``e2e`` is the same through ``Engine.generate``'s own step loop with host
token ids in and out; ``prefill`` is a 2,048-token prompt in one step; ``roofline`` compares the bytes
a decode step must read with the measured copy bandwidth; ``points`` are decode rates at batch 1 and 64.
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

# The layer sizes of Qwen3-8B, the model the reference quotes its decode throughput on.
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
    runner = eng.runner
    vocab = config["vocab_size"]
    gen = torch.Generator().manual_seed(1)

    def prompt():
        return torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()

    # bytes and flops of the model, from the configuration
    H, I, L = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    nh, nkv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    layer_params = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I
    weight_bytes = 2 * (L * layer_params + vocab * H)
    kv_bytes_per_token = 2 * L * nkv * d * 2

    def decode_steps(batch: int, steps: int, warmup: int):
        """(ms per step, launches per step): `batch` requests with PROMPT_LEN tokens cached, then timed decode steps."""
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
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            one()
        t1.record()
        torch.cuda.synchronize()
        launches = (kernels.launch_count() - n0) / steps
        for r in rids:
            runner.release(r)
        return t0.elapsed_time(t1) / steps, launches

    clocks = ClockSampler(args.clock_interval_ms)
    clocks.start()
    time.sleep(0.3)
    lo = clocks.mark()
    ms, launches = decode_steps(args.batch, args.steps, args.warmup)
    hi = clocks.mark()
    value = args.batch * 1e3 / ms
    ctx_mid = PROMPT_LEN + args.warmup + args.steps / 2
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # end to end: the engine's own loop, host token ids in, host token ids out, every step
    sp = SamplingParams.greedy(max_tokens=args.steps + args.warmup + 16, ignore_eos=True)  # none ends inside the timed loop
    for _ in range(args.batch):
        eng.add_request(prompt(), sp)
    reqs = list(eng.scheduler.waiting)
    while any(not r.output for r in reqs):
        eng.step()
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_e2e = 0
    for _ in range(args.steps - 1):
        if not eng.has_work():
            break
        eng.step()
        n_e2e += 1
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / max(n_e2e, 1)
    while eng.has_work():
        eng.step()
    # the step's description as it is copied from pinned host memory: the replayed graph's whole fixed buffer
    graphs = runner.graphs
    meta_ints = graphs.captured[graphs.bucket_for(args.batch)].buffer.numel() if graphs is not None else 0

    out = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, 2,048-token prompts cached, 1xB200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_full": FULL_LAYERS, "hidden": H, "heads": nh,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": vocab, "global_batch": args.batch,
                   "seq_len": CONFIG_8B["max_position_embeddings"], "prompt_len": PROMPT_LEN, "block_size": block,
                   "parallelism": "none", "l2": "inputs larger than L2 (weights read once per step)",
                   "sampling": "greedy"},
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": 4 * meta_ints, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(round(launches * args.steps)),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
        "clocks": clocks.summary(lo, hi),
    }

    if not args.no_points:
        # prefill: one 2,048-token prompt in one step
        times = []
        for i in range(5):
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
        gemm_flops = 2 * PROMPT_LEN * L * layer_params + 2 * vocab * H
        attn_flops = L * 4 * nh * d * PROMPT_LEN * (PROMPT_LEN + 1) / 2
        flops = gemm_flops + attn_flops
        out["prefill"] = {"value": round(PROMPT_LEN * 1e3 / pms, 1), "tokens": PROMPT_LEN, "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "tflops": round(flops / (pms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
                          "of": pk["source"]}
        if pk.get("bf16_tflops_sustained"):
            # the same library product back to back for seconds, under the power cap: what a step of tens of
            # milliseconds can be compared with; "frac" stays the fraction of the burst figure
            out["prefill"]["frac_of_sustained"] = round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        points = {}
        for b in (1, 64):
            pms_b, _ = decode_steps(b, 64 if b == 64 else 128, 4)
            points[f"decode_b{b}"] = round(b * 1e3 / pms_b, 1)
        out["points"] = points
    clocks.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
