"""Trace replay: drive the step function with given token ids and write logits to disk.

It has no forward pass, cache or loader of its own: it loads the model as generation does, and
every step goes through :meth:`ModelRunner.step`.  The reference has no such tool; its nearest
relative is the benchmark loop (inferrs/src/engine.rs:2557-2641).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

from ..cache.manager import CacheError
from ..runtime import Runtime
from .batch import BatchError, StepEntry
from .loading import load_model_dir
from .runner import ModelRunner

TOKEN_ROUNDING = 64  # --max-tokens counts every request's tokens rounded up to this


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time, each request's count rounded up to 64")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--max-requests", type=int, default=8, help="most requests that are live at a time")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if args.block_size <= 0 or TOKEN_ROUNDING % args.block_size:
        ap.error(f"--block-size must divide {TOKEN_ROUNDING}")

    rt = Runtime.cuda(args.dtype)
    spec, weights, _ = load_model_dir(args.model, rt)
    n_tokens = (args.max_tokens + TOKEN_ROUNDING - 1) // TOKEN_ROUNDING * TOKEN_ROUNDING
    runner = ModelRunner(spec, weights, rt, page_size=args.block_size, n_pages=n_tokens // args.block_size,
                         max_requests=args.max_requests)
    os.makedirs(args.out, exist_ok=True)

    for line_no, line in enumerate(sys.stdin, 1):
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
            ends = rec.get("end", [])
        except (ValueError, KeyError, TypeError) as e:
            print(f"trace_run: line {line_no} is not a step: {e}", file=sys.stderr)
            return 2
        if entries:
            # A step that the cache cannot hold (more tokens than --max-tokens allows, more requests than
            # --max-requests) or that is no step (a token outside the vocabulary, a wanted place outside the
            # tokens) ends the replay with status 3 and one line that says why; the cache is as it was before it.
            admitted = []
            try:
                for e in entries:
                    if not runner.has(e.rid):
                        runner.admit(e.rid)
                        admitted.append(e.rid)
                logits = runner.step(entries)
            except (CacheError, BatchError, ValueError) as e:
                for rid in admitted:
                    runner.release(rid)
                print(f"trace_run: step {step}: {e}", file=sys.stderr)
                return 3
            if logits.shape[0] > 0:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f"{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in ends:
            if runner.has(rid):
                runner.release(rid)
        print(f"done {step}", flush=True)
    return 0
