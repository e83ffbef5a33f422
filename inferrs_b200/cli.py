"""Command line in the manner of the reference's ``inferrs run`` and ``inferrs bench``.

Option names, meanings and defaults are the reference's where it has them
(inferrs/src/main.rs:91-204 shared options, inferrs/src/run.rs:34-146 ``run``,
inferrs/src/bench.rs:21-38 ``bench``).  The model is a local folder (the reference's
``load_local_model`` contract, inferrs/src/hub.rs:28-85).  Prompts are token ids: text needs a
``tokenizer.json`` in the model folder and the ``tokenizers`` library.

    python -m inferrs_b200 run MODEL_DIR --prompt-ids 1,2,3 --max-tokens 32 --temperature 0
    python -m inferrs_b200 run CONFIG.json --random-weights 0 --random-prompt 64 --ignore-eos --max-tokens 32
    python -m inferrs_b200 bench MODEL_DIR --prompt-len 128 --max-tokens 128
    python -m inferrs_b200 replay --model MODEL_DIR --dtype bfloat16 --out DIR --max-tokens 256 < steps.jsonl

(``replay`` is the trace replay program, ``bin/trace_run``, under this command's roof: ``engine/trace.py``.)

Beyond the reference's options: ``--prefill-chunk`` (the most tokens of one prompt in a step), ``--ignore-eos``,
``--min-p``, ``--random-weights SEED`` (the model argument is then a config.json, or a folder with one, and the
weights are made on the device), ``--random-prompt LEN`` and ``--prompt-file``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from typing import List, Optional


def _shared(ap: argparse.ArgumentParser):
    ap.add_argument("model", help="folder with config.json and model.safetensors (or *.safetensors shards)")
    ap.add_argument("--dtype", default="bf16", help="weight and activation type: bf16 or f32 (default bf16)")
    ap.add_argument("--max-seq-len", type=int, default=0, help="maximum sequence length (0 = model default)")
    ap.add_argument("--block-size", type=int, default=16, help="KV cache block size in tokens")
    ap.add_argument("--max-blocks", type=int, default=0,
                    help="KV cache blocks (0 = sized by --paged-attention)")
    ap.add_argument("--max-batch-size", type=int, default=32, help="maximum concurrent sequences")
    ap.add_argument("--max-tokens-per-step", type=int, default=2048, help="token budget per scheduler step")
    ap.add_argument("--paged-attention", type=float, default=0.9, metavar="FRACTION",
                    help="fraction of free device memory reserved for paged KV blocks")
    ap.add_argument("--temperature", type=float, default=0.7, help="sampling temperature")
    ap.add_argument("--top-p", type=float, default=0.9, help="nucleus sampling threshold")
    ap.add_argument("--top-k", type=int, default=50, help="top-k sampling (0 = off)")
    ap.add_argument("--max-tokens", type=int, default=2048, help="max tokens to generate")
    ap.add_argument("--seed", type=int, default=None, help="seed for reproducible sampling")
    ap.add_argument("--min-p", type=float, default=0.0, help="keep tokens with p >= min_p * p_max (0 = off)")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at end-of-sequence or stop tokens")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="most tokens of one prompt in a step (0 = the step's whole budget)")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="MODEL is a config.json (or a folder with one): weights are random, N(0, 0.02), from this seed")


def _engine(args):
    from .engine.engine import Engine
    common = dict(dtype=args.dtype, block_size=args.block_size, num_blocks=args.max_blocks or None,
                  paged_attention=args.paged_attention, max_batch_size=args.max_batch_size,
                  max_tokens_per_step=args.max_tokens_per_step, max_seq_len=args.max_seq_len,
                  prefill_chunk=args.prefill_chunk or None)
    if args.random_weights is not None:
        path = os.path.join(args.model, "config.json") if os.path.isdir(args.model) else args.model
        with open(path, "r", encoding="utf-8") as f:
            config = json.load(f)
        return Engine(config=config, random_weights=args.random_weights, **common)
    return Engine(args.model, **common)


def _tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def cmd_run(args) -> int:
    from .sampling.params import SamplingParams
    tok = _tokenizer(args.model) if os.path.isdir(args.model) else None
    eng = None
    prompt_text = args.prompt
    if args.prompt_file is not None:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            content = f.read()
        if all(t.lstrip("-").isdigit() for t in content.replace(",", " ").split()) and content.strip():
            args.prompt_ids = content          # a file of token ids
        else:
            prompt_text = content
    if args.random_prompt:
        import random
        eng = _engine(args)
        rng = random.Random(args.seed if args.seed is not None else 0)
        ids = [rng.randrange(eng.spec.vocab_size) for _ in range(args.random_prompt)]
        args.prompt_ids = " ".join(map(str, ids))
    elif args.prompt_ids:
        ids = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    elif prompt_text is not None:
        if tok is None:
            print("run: a text prompt needs tokenizer.json in the model folder and the tokenizers library; "
                  "use --prompt-ids", file=sys.stderr)
            return 2
        text = prompt_text if args.system is None else args.system + "\n" + prompt_text
        ids = tok.encode(text).ids
    else:
        print("run: give a prompt, --prompt-ids, --prompt-file or --random-prompt", file=sys.stderr)
        return 2
    eng = eng or _engine(args)
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                        repetition_penalty=args.repetition_penalty, repeat_last_n=args.repeat_last_n,
                        frequency_penalty=args.frequency_penalty, max_tokens=args.max_tokens, seed=args.seed,
                        ignore_eos=args.ignore_eos)
    t0 = time.perf_counter()
    out: List[int] = []
    text = ""
    for t in eng.stream(ids, sp):        # printed as it comes
        out.append(t)
        if tok is not None and not args.prompt_ids:
            whole = tok.decode(out)
            print(whole[len(text):], end="", flush=True)
            text = whole
        else:
            print(t, end=" ", flush=True)
    print()
    dt = time.perf_counter() - t0
    print(f"[{len(ids)} prompt tokens, {len(out)} generated, finish={eng.last_streamed.finish_reason}, {dt:.2f} s]",
          file=sys.stderr)
    return 0


def cmd_bench(args) -> int:
    """Prefill and decode rates for one sequence, as ``inferrs bench`` measures them
    (inferrs/src/bench.rs:53-221, inferrs/src/engine.rs:2557-2641): a synthetic prompt of
    ``--prompt-len`` equal tokens, stop tokens bypassed, ``--warmup`` + ``--runs`` runs."""
    import torch
    from .sampling.params import SamplingParams
    eng = _engine(args)
    prompt = [1 % eng.spec.vocab_size] * args.prompt_len
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                        max_tokens=args.max_tokens, seed=args.seed if args.seed is not None else 0, ignore_eos=True)
    prefill, decode, ttft, e2e = [], [], [], []
    for run in range(args.warmup + args.runs):
        eng.add_request(prompt, sp)
        req = eng.scheduler.waiting[-1]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done, first = None, None
        while done is None:
            fin = eng.step()
            torch.cuda.synchronize()
            if first is None and req.output:
                first = time.perf_counter()
            done = fin[0] if fin else None
        t1 = time.perf_counter()
        if run >= args.warmup:
            n_out = len(done.output)
            prefill.append(args.prompt_len / (first - t0))
            decode.append(max(n_out - 1, 1) / max(t1 - first, 1e-9))
            ttft.append((first - t0) * 1e3)
            e2e.append((t1 - t0) * 1e3)
    mean = statistics.mean
    sd = lambda v: statistics.stdev(v) if len(v) > 1 else 0.0  # noqa: E731
    q = lambda v, p: sorted(v)[min(len(v) - 1, int(p * len(v)))]  # noqa: E731
    out = {"prompt_len": args.prompt_len, "max_tokens": args.max_tokens, "runs": args.runs,
           "prefill_tok_s": mean(prefill), "prefill_tok_s_sd": sd(prefill),
           "decode_tok_s": mean(decode), "decode_tok_s_sd": sd(decode),
           "ttft_ms": mean(ttft), "e2e_ms_p50": q(e2e, 0.5), "e2e_ms_p90": q(e2e, 0.9)}
    print(json.dumps(out))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["replay"]:
        # the trace replay program under this command's roof: the same options as bin/trace_run, steps on standard input
        from .engine.trace import main as replay
        return replay(argv[1:])
    ap = argparse.ArgumentParser(prog="inferrs_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="generate from one prompt and exit")
    _shared(run)
    run.add_argument("prompt", nargs="?", default=None, help="text prompt (needs tokenizer.json)")
    run.add_argument("--prompt-ids", default=None, help="prompt as token ids, separated by commas or spaces")
    run.add_argument("--prompt-file", default=None, help="file with the prompt: token ids, or text")
    run.add_argument("--random-prompt", type=int, default=0, metavar="LEN",
                     help="a prompt of LEN token ids drawn uniformly from the vocabulary (seeded by --seed)")
    run.add_argument("--system", default=None, help="system prompt, put before the prompt")
    run.add_argument("--repetition-penalty", type=float, default=1.1, help="llama.cpp-style; 1.0 = disabled")
    run.add_argument("--repeat-last-n", type=int, default=64, help="window of the penalties; 0 = disabled")
    run.add_argument("--frequency-penalty", type=float, default=0.0, help="OpenAI-style; 0.0 = disabled")
    run.set_defaults(fn=cmd_run)
    bench = sub.add_parser("bench", help="benchmark prefill and decode of one sequence")
    _shared(bench)
    bench.add_argument("--warmup", type=int, default=1, help="warm-up runs (discarded)")
    bench.add_argument("--runs", type=int, default=5, help="timed runs")
    bench.add_argument("--prompt-len", type=int, default=128, help="synthetic prompt tokens")
    bench.set_defaults(fn=cmd_bench)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
