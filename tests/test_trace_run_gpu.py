"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3
from helpers import CONFIG_A, CONFIG_B, CONFIG_D, cut, random_tokens, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(model_dir, dtype, steps, out_dir, max_tokens):
    """Feed the steps one at a time, waiting for ``done <step>`` after each, as the contract says."""
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype",
                          dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {s['step']}", line
    p.stdin.close()
    assert p.wait(timeout=120) == 0


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype,name", [("float32", "B"), ("bfloat16", "B"), ("bfloat16", "D")])
def test_replay_mixed_trace(model_dirs, tmp_path, dtype, name):
    cfg = CONFIG_B if name == "B" else CONFIG_D
    vocab = cfg["vocab_size"]
    lens = {"a": 90, "b": 37, "c": 64, "d": 120, "e": 50}
    toks = {k: random_tokens(n, vocab, seed=ord(k)) for k, n in lens.items()}
    store = None if dtype == "float32" else torch.bfloat16
    mcfg, w = plain_qwen3.read_model(model_dirs[name])
    want = {k: plain_qwen3.forward(mcfg, w, t, store=store) for k, t in toks.items()}
    # a, b, c, d start; e comes when b has ended and takes over its pages (320 tokens of cache in all)
    at = {k: 0 for k in lens}
    live, waiting = ["a", "b", "c", "d"], ["e"]
    sizes = [11, 2, 5, 1, 30, 3, 1, 1]
    steps, where = [], []
    i = 0
    while live:
        entries, ends = [], []
        for j, k in enumerate(list(live)):
            if (i + j) % 4 == 3 and len(live) > 1:
                continue
            n = min(sizes[(i + j) % len(sizes)], lens[k] - at[k])
            want_rows = list(range(n)) if (i + j) % 2 == 0 else [n - 1]
            entries.append({"id": k, "tokens": toks[k][at[k]:at[k] + n], "want": want_rows})
            where.append((len(steps), k, [at[k] + r for r in want_rows]))
            at[k] += n
            if at[k] == lens[k]:
                ends.append(k)
        steps.append({"step": len(steps), "entries": entries, "end": ends})
        for k in ends:
            live.remove(k)
            if waiting:
                live.append(waiting.pop(0))
        i += 1
    out_dir = str(tmp_path / "out")
    replay(model_dirs[name], dtype, steps, out_dir, max_tokens=128 + 64 + 64 + 128)
    got = {s: read(out_dir, s, vocab) for s in {w[0] for w in where}}
    offset = {}
    worst = 0.0
    for s, k, rows in where:
        o = offset.get(s, 0)
        worst = max(worst, rel_err(got[s][o:o + len(rows)], want[k][rows]))
        offset[s] = o + len(rows)
    assert worst < (1e-4 if dtype == "float32" else 3e-2), worst


def test_step_without_wanted_rows_writes_no_file(model_dirs, tmp_path):
    toks = random_tokens(20, CONFIG_A["vocab_size"], seed=1)
    steps = [{"step": 0, "entries": [{"id": 1, "tokens": toks[:12], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": 1, "tokens": toks[12:], "want": [7]}], "end": [1]}]
    out_dir = str(tmp_path / "o")
    replay(model_dirs["A"], "float32", steps, out_dir, max_tokens=64)
    assert sorted(os.listdir(out_dir)) == ["1.f32"]
    mcfg, w = plain_qwen3.read_model(model_dirs["A"])
    assert rel_err(read(out_dir, 1, CONFIG_A["vocab_size"])[0], plain_qwen3.forward(mcfg, w, toks)[19]) < 1e-4


def test_a_step_that_does_not_fit_ends_the_replay_with_a_status(model_dirs, tmp_path):
    """More tokens than --max-tokens gives pages for: the step before is answered, the step that does not fit is
    not; the program says why on standard error and exits with status 3 (no traceback)."""
    toks = random_tokens(200, CONFIG_A["vocab_size"], seed=2)
    out_dir = str(tmp_path / "o")
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["A"], "--dtype",
                          "float32", "--out", out_dir, "--max-tokens", "128"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:100], "want": [99]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": toks[100:160], "want": [0]}], "end": []}]
    out, err = p.communicate("".join(json.dumps(s) + "\n" for s in steps), timeout=300)
    assert p.returncode == 3, (p.returncode, err[-500:])
    assert out.split("\n")[0] == "done 0" and "done 1" not in out
    assert "trace_run: step 1:" in err and "Traceback" not in err
    assert sorted(os.listdir(out_dir)) == ["0.f32"]


def test_the_replay_subcommand_is_the_same_program(model_dirs, tmp_path):
    """``python -m inferrs_b200 replay`` takes the options and the steps of ``bin/trace_run`` and writes the same bytes."""
    toks = random_tokens(24, CONFIG_A["vocab_size"], seed=3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:17], "want": [16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[17:], "want": [0, 6]}], "end": ["a"]}]
    one, two = str(tmp_path / "one"), str(tmp_path / "two")
    replay(model_dirs["A"], "float32", steps, one, max_tokens=64)
    p = subprocess.run([sys.executable, "-m", "inferrs_b200", "replay", "--model", model_dirs["A"], "--dtype", "float32",
                        "--out", two, "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-500:]
    assert p.stdout.split() == ["done", "0", "done", "1"]
    for name in ("0.f32", "1.f32"):
        with open(os.path.join(one, name), "rb") as a, open(os.path.join(two, name), "rb") as b:
            assert a.read() == b.read()
