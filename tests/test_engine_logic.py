"""The engine's own logic (batches, cache, steps) on the CPU, with the plain kernel statements of
``kernel_refs`` in the kernels' place: every way of cutting must give the plain model's logits."""
import pytest
import torch

import kernel_refs
import plain_qwen3
from helpers import CONFIG_A, CONFIG_B, PAGE_SIZE, cut, random_tokens, rel_err
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.engine.loading import load_model_dir
from inferrs_b200.engine.runner import ModelRunner
from inferrs_b200.runtime import Runtime


def make_runner(model_dir, page_size, n_pages, max_requests=4, dtype=torch.float32):
    rt = Runtime(device=torch.device("cpu"), dtype=dtype)
    spec, weights, _ = load_model_dir(model_dir, rt)
    return ModelRunner(spec, weights, rt, page_size=page_size, n_pages=n_pages, max_requests=max_requests)


def plain_logits(model_dir, tokens):
    cfg, w = plain_qwen3.read_model(model_dir)
    return plain_qwen3.forward(cfg, w, tokens)


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt(model_dirs, monkeypatch, name):
    kernel_refs.install(monkeypatch)
    cfg = CONFIG_A if name == "A" else CONFIG_B
    toks = random_tokens(45, cfg["vocab_size"], seed=1)
    runner = make_runner(model_dirs[name], PAGE_SIZE[name], n_pages=64)
    runner.admit("a")
    got = runner.step([StepEntry("a", toks, list(range(len(toks))))])
    assert rel_err(got, plain_logits(model_dirs[name], toks)) < 1e-4


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_decode(model_dirs, monkeypatch, name):
    kernel_refs.install(monkeypatch)
    cfg = CONFIG_A if name == "A" else CONFIG_B
    toks = random_tokens(61, cfg["vocab_size"], seed=5)
    want = plain_logits(model_dirs[name], toks)
    runner = make_runner(model_dirs[name], PAGE_SIZE[name], n_pages=32)
    runner.admit("a")
    rows, at = [], 0
    for n in cut(len(toks) - 8, [7, 2, 13, 3, 2]) + [1] * 8:
        rows.append(runner.step([StepEntry("a", toks[at:at + n], list(range(n)))]))
        at += n
    assert rel_err(torch.cat(rows), want) < 1e-4


def test_mixed_with_page_reuse(model_dirs, monkeypatch):
    kernel_refs.install(monkeypatch)
    name, cfg = "B", CONFIG_B
    lens = [40, 23, 57, 31, 18, 44]
    prompts = [random_tokens(n, cfg["vocab_size"], seed=10 + i) for i, n in enumerate(lens)]
    want = [plain_logits(model_dirs[name], p) for p in prompts]
    # 4 live requests of at most 57 tokens need 4 * 4 pages of 16: later requests reuse freed pages
    runner = make_runner(model_dirs[name], PAGE_SIZE[name], n_pages=14)
    got = [[] for _ in prompts]
    at = [0] * len(prompts)
    live, nxt, step = [], 0, 0
    sizes = [5, 2, 9, 1, 3, 16, 1, 1]
    while live or nxt < len(prompts):
        while len(live) < 4 and nxt < len(prompts):
            need = sum((lens[i] + 15) // 16 for i in live) + (lens[nxt] + 15) // 16
            if need > 14:
                break
            runner.admit(nxt)
            live.append(nxt)
            nxt += 1
        entries = []
        for k, i in enumerate(live):
            if (step + k) % 3 == 2 and len(live) > 1:
                continue  # this request sits the step out
            n = min(sizes[(step + i) % len(sizes)], lens[i] - at[i])
            entries.append((i, n))
        if not entries:
            entries = [(live[0], 1)]
        out = runner.step([StepEntry(i, prompts[i][at[i]:at[i] + n], list(range(n))) for i, n in entries])
        o = 0
        for i, n in entries:
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
        for i in [i for i in live if at[i] == lens[i]]:
            runner.release(i)
            live.remove(i)
        runner.manager.check_invariants()
        step += 1
    for i in range(len(prompts)):
        assert rel_err(torch.cat(got[i]), want[i]) < 1e-4, i
