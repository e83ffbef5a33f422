"""Generation through the Python entry point on the CPU (plain kernel statements in the kernels' place)
against a plain loop: forward the whole sequence, pick the next token, append."""
import pytest
import torch

import kernel_refs
import plain_qwen3
import plain_sampler
from helpers import CONFIG_A, CONFIG_B, PAGE_SIZE, random_tokens
from inferrs_b200.engine.engine import Engine
from inferrs_b200.runtime import Runtime
from inferrs_b200.sampling.params import SamplingParams, uniform_for


def plain_generate(model_dir, prompt, n, **sampling):
    cfg, w = plain_qwen3.read_model(model_dir)
    toks = list(prompt)
    for _ in range(n):
        logits = plain_qwen3.forward(cfg, w, toks)[-1]
        toks.append(plain_sampler.sample_token(logits.numpy(), toks, **sampling))
    return toks[len(prompt):]


def cpu_engine(model_dir, name, **kw):
    return Engine(model_dir, block_size=PAGE_SIZE[name], runtime=Runtime(torch.device("cpu"), torch.float32), **kw)


def test_uniform_matches_the_plain_generator():
    for seed, step in [(0, 0), (4, 17), (2 ** 63 - 1, 5000), (123456789, 1)]:
        assert abs(uniform_for(seed, step) - float(plain_sampler.rand_f32(seed, step))) < 1e-7


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation(model_dirs, monkeypatch, name):
    kernel_refs.install(monkeypatch)
    cfg = CONFIG_A if name == "A" else CONFIG_B
    prompts = [random_tokens(n, cfg["vocab_size"], seed=40 + n) for n in (5, 17, 33)]
    eng = cpu_engine(model_dirs[name], name, num_blocks=64, max_batch_size=4, max_tokens_per_step=24)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=8))
    for p, g in zip(prompts, got):
        assert g == plain_generate(model_dirs[name], p, 8, temperature=0.0, repetition_penalty=1.0)
    assert eng.stats()["free_pages"] == eng.stats()["pages"]


def test_sampled_generation_matches_the_plain_sampler(model_dirs, monkeypatch):
    kernel_refs.install(monkeypatch)
    name, cfg = "B", CONFIG_B
    prompts = [random_tokens(n, cfg["vocab_size"], seed=50 + n) for n in (1, 9, 40)]
    opts = dict(temperature=0.8, top_k=20, top_p=0.95, repetition_penalty=1.1, repeat_last_n=16,
                frequency_penalty=0.2, presence_penalty=0.1, min_p=0.01)
    eng = cpu_engine(model_dirs[name], name, num_blocks=32, max_batch_size=4, max_tokens_per_step=7)
    got = eng.generate(prompts, SamplingParams(max_tokens=10, seed=4, **opts))
    for p, g in zip(prompts, got):
        assert g == plain_generate(model_dirs[name], p, 10, seed=4, **opts)


def test_preemption_gives_the_same_tokens(model_dirs, monkeypatch):
    kernel_refs.install(monkeypatch)
    name, cfg = "A", CONFIG_A
    prompts = [random_tokens(n, cfg["vocab_size"], seed=60 + n) for n in (9, 14, 11)]
    sp = SamplingParams(temperature=0.9, top_k=0, top_p=1.0, repetition_penalty=1.0, max_tokens=14, seed=7)
    roomy = cpu_engine(model_dirs[name], name, num_blocks=64, max_batch_size=4)
    want = roomy.generate(prompts, sp)
    tight = cpu_engine(model_dirs[name], name, num_blocks=14, max_batch_size=4)   # 14 pages of 4 tokens
    got = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    assert got == want
