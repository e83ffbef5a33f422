"""The sampling kernels against the plain host sampler (written from the reference's), and generation
through the Python entry point against a plain loop."""
import numpy as np
import pytest
import torch

import plain_qwen3
import plain_sampler
from helpers import CONFIG_A, CONFIG_B, PAGE_SIZE, random_tokens
from inferrs_b200.sampling.params import SamplingParams

pytestmark = pytest.mark.gpu


def _logits(rows, vocab, seed, spread=3.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn((rows, vocab), generator=g) * spread


@pytest.mark.parametrize("vocab", [517, 5000, 151936])
@pytest.mark.parametrize("opts", [
    dict(temperature=0.8, top_k=0, top_p=1.0, min_p=0.0),
    dict(temperature=0.7, top_k=50, top_p=0.9, min_p=0.0),
    dict(temperature=1.3, top_k=0, top_p=0.6, min_p=0.0),
    dict(temperature=1.0, top_k=7, top_p=1.0, min_p=0.2),
    dict(temperature=0.0, top_k=50, top_p=0.9, min_p=0.0),
])
def test_sample_kernel_matches_plain_sampler(vocab, opts):
    from inferrs_b200.sampling.sampler import Sampler
    rows = 12
    logits = _logits(rows, vocab, seed=vocab % 97)
    logits[3, 10] = logits[3, 200] = logits[3].max() + 1.0     # equal probabilities: lowest id first
    hist = [list(range(5 + r)) for r in range(rows)]
    sp = SamplingParams(repetition_penalty=1.0, max_tokens=4, seed=None, **opts)
    seeds = [100 + r for r in range(rows)]
    got = Sampler(torch.device("cuda")).sample(logits.cuda(), [sp] * rows, seeds, hist).cpu().tolist()
    # a walk over the whole vocabulary is compared with the plain sampler's exact sums: see its docstring
    precise = opts["top_k"] == 0 and opts["top_p"] == 1.0 and vocab > 1000
    want = [plain_sampler.sample_token(logits[r].numpy(), hist[r], repetition_penalty=1.0, seed=seeds[r],
                                       precise=precise, **opts) for r in range(rows)]
    assert got == want


@pytest.mark.parametrize("vocab", [263, 5000, 151936])
def test_a_row_shared_by_one_to_eight_ctas_gives_the_same_token(vocab):
    """The selection kernel cuts a row's vocabulary over a cluster of CTAs when there are few rows: whatever the
    cluster, every row gets the token that the plain selection gives (rows with every option, equal probabilities,
    a row of one value, greedy rows; top-k with few survivors, which the kernel keeps as a list, and with many)."""
    import kernel_refs as R
    from inferrs_b200 import kernels as K
    rows = 10
    logits = _logits(rows, vocab, seed=11).cuda()
    logits[3, 10] = logits[3, 200] = logits[3].max() + 1.0
    logits[4, :] = 0.25                                        # all equal: the walk counts token ids
    temperature = torch.tensor([0.8, 0.7, 1.3, 1.0, 1.0, 0.0, 0.7, 2.0, 0.7, 0.5]).cuda()
    # (1,000 survivors of top-k are few enough for the kernel's list in shared memory, 3,000 are not)
    top_k = torch.tensor([0, 50, 3000, 7, 0, 50, 1, 0, 1000, 3], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 0.9, 0.6, 1.0, 1.0, 0.9, 1.0, 0.999, 0.5, 1.0]).cuda()
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.2, 0.0, 0.0, 0.0, 0.0, 0.01, 0.0]).cuda()
    # rows that walk the whole of a large vocabulary are left out of the comparison with the plain selection: far
    # down the tail the kernel's fixed-point masses and the plain float64 sums part (see plain_sampler's docstring)
    exact = [r for r in range(rows) if vocab < 1000 or r not in (0, 7)]
    for draw in (0.0, 0.37, 0.999999):
        uniform = torch.full((rows,), draw).cuda()
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        R.sample(logits, temperature, top_k, top_p, min_p, uniform, want)
        alone = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        K.sample(logits, temperature, top_k, top_p, min_p, uniform, alone, cluster=1)
        assert [alone.tolist()[r] for r in exact] == [want.tolist()[r] for r in exact], f"draw {draw}"
        for cluster in (2, 4, 8, 0):
            got = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
            K.sample(logits, temperature, top_k, top_p, min_p, uniform, got, cluster=cluster)
            assert got.tolist() == alone.tolist(), f"cluster {cluster}, draw {draw}"
    with pytest.raises(K.KernelError):
        K.sample(logits, temperature, top_k, top_p, min_p, uniform, got, cluster=3)


def test_penalties_and_mixed_rows():
    from inferrs_b200.sampling.sampler import Sampler
    vocab, rows = 2000, 6
    logits = _logits(rows, vocab, seed=5)
    hist = [random_tokens(30 + 7 * r, vocab, seed=r) + [3, 3, 3] for r in range(rows)]
    params = [SamplingParams(temperature=0.9, top_k=40, top_p=0.95, repetition_penalty=1.3, repeat_last_n=16,
                             frequency_penalty=0.5, presence_penalty=0.25, max_tokens=1),
              SamplingParams.greedy(),
              SamplingParams(temperature=0.0, repetition_penalty=5.0, repeat_last_n=64, max_tokens=1),
              SamplingParams(temperature=1.1, top_k=0, top_p=1.0, repetition_penalty=1.0, max_tokens=1),
              SamplingParams(temperature=0.5, repeat_last_n=0, max_tokens=1),
              SamplingParams(temperature=0.7, max_tokens=1)]
    logits[2, 3] = logits[2].max() + 1.0     # the greedy row's favourite was seen: the penalty must move it
    seeds = list(range(rows))
    got = Sampler(torch.device("cuda")).sample(logits.cuda(), params, seeds, hist).cpu().tolist()
    want = []
    for r, p in enumerate(params):
        want.append(plain_sampler.sample_token(
            logits[r].numpy(), hist[r], temperature=p.temperature, top_p=p.top_p, top_k=p.top_k,
            repetition_penalty=p.repetition_penalty, repeat_last_n=p.repeat_last_n,
            frequency_penalty=p.frequency_penalty, presence_penalty=p.presence_penalty, min_p=p.min_p, seed=seeds[r]))
    assert got == want
    assert got[2] != 3


def test_sampling_follows_the_distribution():
    from inferrs_b200 import kernels as K
    probs = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    n = 4000
    logits = probs.log().repeat(n, 1).cuda().contiguous()
    u = torch.rand(n, generator=torch.Generator().manual_seed(0)).cuda()
    one, zero = torch.ones(n, device="cuda"), torch.zeros(n, device="cuda")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    K.sample(logits, one, torch.zeros(n, dtype=torch.int32, device="cuda"), one, zero, u, out)
    freq = torch.bincount(out.long().cpu(), minlength=5).float() / n
    assert float((freq - probs).abs().max()) < 0.03


def _plain_generate(model_dir, prompt, n, **sampling):
    cfg, w = plain_qwen3.read_model(model_dir)
    toks = list(prompt)
    for _ in range(n):
        logits = plain_qwen3.forward(cfg, w, toks)[-1]
        toks.append(plain_sampler.sample_token(logits.numpy(), toks, **sampling))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name):
    from inferrs_b200 import Engine
    cfg = CONFIG_A if name == "A" else CONFIG_B
    prompts = [random_tokens(n, cfg["vocab_size"], seed=70 + n) for n in (5, 17, 33)]
    eng = Engine(model_dirs[name], dtype="f32", block_size=PAGE_SIZE[name], num_blocks=64, max_batch_size=4,
                 max_tokens_per_step=24)
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=16))
    for p, g in zip(prompts, got):
        assert g == _plain_generate(model_dirs[name], p, 16, temperature=0.0, repetition_penalty=1.0)
    bf = Engine(model_dirs[name], dtype="bf16", block_size=PAGE_SIZE[name], num_blocks=64, max_batch_size=4)
    out = bf.generate(prompts, SamplingParams.greedy(max_tokens=16))
    assert all(len(o) == 16 for o in out)
    assert bf.stats()["free_pages"] == bf.stats()["pages"]


def test_sampled_generation_in_portions_with_preemption(model_dirs):
    """Configuration B: prompts of 1/9/40/100 tokens in portions of 7 beside decoding, temperature 0.8, seed 4,
    with so few pages that the youngest request is preempted and recomputed."""
    from inferrs_b200 import Engine
    name, cfg = "B", CONFIG_B
    prompts = [random_tokens(n, cfg["vocab_size"], seed=80 + n) for n in (1, 9, 40, 100)]
    opts = dict(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0)
    sp = SamplingParams(max_tokens=24, seed=4, **opts)
    eng = Engine(model_dirs[name], dtype="f32", block_size=16, num_blocks=13, max_batch_size=4,
                 max_tokens_per_step=12, prefill_chunk=7)
    got = eng.generate(prompts, sp)
    assert eng.stats()["preemptions"] > 0
    for p, g in zip(prompts, got):
        assert g == _plain_generate(model_dirs[name], p, 24, seed=4, **opts)


def test_warm_up_captures_every_batch_size_and_changes_nothing(model_dirs):
    """Graphs captured before the first request (with stand-in requests that are released again) give the
    tokens that graphs captured on demand give; the cache is whole afterwards."""
    from inferrs_b200 import Engine
    prompts = [random_tokens(n, CONFIG_B["vocab_size"], seed=90 + n) for n in (3, 12, 21)]
    kw = dict(dtype="f32", block_size=PAGE_SIZE["B"], num_blocks=64, max_batch_size=6)
    cold = Engine(model_dirs["B"], **kw)
    want = cold.generate(prompts, SamplingParams.greedy(max_tokens=12))
    warm = Engine(model_dirs["B"], **kw)
    assert warm.warm_up([3]) == [4]
    assert warm.warm_up() == [1, 2, 6, -32, -64, -128, -256, -512, -1024]   # row counts that the context of 640 reaches
    assert warm.warm_up() == []
    warm.runner.manager.check_invariants()
    assert warm.stats()["free_pages"] == warm.stats()["pages"]
    assert warm.generate(prompts, SamplingParams.greedy(max_tokens=12)) == want
    assert sorted(warm.runner.graphs.captured) == [1, 2, 4, 6]


@pytest.mark.parametrize("name,dtype", [("B", "f32"), ("D", "bf16")])
def test_steps_launched_one_ahead_give_the_same_tokens(model_dirs, name, dtype):
    """With ``overlap`` a decode step is launched before the host has read the tokens of the step before it (the
    device hands them on).  Greedy and seeded sampling, requests that stop at a token nobody could foresee, and
    a cache so small that requests are preempted must all give what the engine gives step by step."""
    from inferrs_b200 import Engine
    cfg = CONFIG_B if name == "B" else __import__("helpers").CONFIG_D
    prompts = [random_tokens(n, cfg["vocab_size"], seed=40 + n) for n in (5, 17, 33, 60)]
    kw = dict(dtype=dtype, block_size=16, num_blocks=64, max_batch_size=4, max_tokens_per_step=48)

    def both(params, **more):
        a = Engine(model_dirs[name], overlap=False, **dict(kw, **more))
        b = Engine(model_dirs[name], overlap=True, **dict(kw, **more))
        assert b.overlap and not a.overlap
        ra = a.generate(prompts, params, return_requests=True)
        rb = b.generate(prompts, params, return_requests=True)
        assert [r.output for r in ra] == [r.output for r in rb]
        assert [r.finish_reason for r in ra] == [r.finish_reason for r in rb]
        assert b.stats()["free_pages"] == b.stats()["pages"] and not b.has_work()
        return ra, b

    ra, b = both(SamplingParams.greedy(max_tokens=40))
    assert b.n_steps_in_vain == 0
    # a token that one of the requests reaches for the first time in the middle of its decoding
    first_seen = [(i, r.output[i]) for r in ra for i in range(4, 36) if r.output[i] not in r.output[:i]
                  and all(r.output[i] not in o.output[:4] for o in ra)]
    assert first_seen, "the test wants a token that first comes up while all requests decode"
    stop = first_seen[0][1]
    ra, b = both(SamplingParams(temperature=0.0, repetition_penalty=1.0, max_tokens=40, stop_token_ids=(stop,)))
    assert any(r.finish_reason == "stop" and 4 < len(r.output) < 40 for r in ra) and b.n_steps_in_vain >= 1
    both(SamplingParams(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0, max_tokens=30, seed=9))
    both(SamplingParams(temperature=0.7, max_tokens=20, seed=3))          # the reference's defaults: penalties
    ra, b = both(SamplingParams.greedy(max_tokens=40), num_blocks=9)      # too few pages for all four at once
    assert b.stats()["preemptions"] > 0


def test_tokens_come_one_by_one_and_through_the_command_line(model_dirs):
    """``Engine.stream`` yields what ``generate`` returns, token by token, also while another request is live;
    the ``run`` command prints the same ids."""
    import subprocess
    import sys
    from helpers import CONFIG_D
    from inferrs_b200 import Engine
    prompt = random_tokens(23, CONFIG_D["vocab_size"], seed=77)
    other = random_tokens(9, CONFIG_D["vocab_size"], seed=78)
    sp = SamplingParams.greedy(max_tokens=14)
    kw = dict(dtype="bf16", block_size=16, num_blocks=32, max_batch_size=4)
    want = Engine(model_dirs["D"], **kw).generate([prompt, other], sp)
    eng = Engine(model_dirs["D"], **kw)
    eng.add_request(other, sp, rid="other")
    got = list(eng.stream(prompt, sp))
    assert got == want[0]
    while eng.has_work():
        eng.step()
    assert eng.stats()["free_pages"] == eng.stats()["pages"]
    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "inferrs_b200", "run", model_dirs["D"], "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "14", "--temperature", "0",
                          "--max-blocks", "32", "--max-batch-size", "4"],
                         cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    # greedy through the command line applies the reference's default repetition penalty: compare with the same
    ref = Engine(model_dirs["D"], **kw).generate([prompt], SamplingParams(temperature=0.0, max_tokens=14))
    assert [int(t) for t in out.stdout.split()] == ref[0]


def test_steps_go_one_ahead_while_requests_wait_for_a_slot(model_dirs):
    """More requests than slots: the waiting ones cannot be let in while all slots are taken, so decode steps still
    go one ahead; the tokens are those of the engine that reads every step's tokens first."""
    from inferrs_b200 import Engine
    prompts = [random_tokens(n, CONFIG_B["vocab_size"], seed=90 + n) for n in (5, 9, 14, 3, 21, 8, 12)]
    params = [SamplingParams.greedy(max_tokens=6 + 3 * i) for i in range(len(prompts))]
    kw = dict(dtype="f32", block_size=16, num_blocks=64, max_batch_size=3, max_tokens_per_step=32)
    a = Engine(model_dirs["B"], overlap=False, **kw)
    b = Engine(model_dirs["B"], overlap=True, **kw)
    assert a.generate(prompts, params) == b.generate(prompts, params)
    # most decode steps of the second engine were launched before the step before them had been read
    assert b.n_steps <= a.n_steps + len(prompts) + b.n_steps_in_vain
    assert b.stats()["free_pages"] == b.stats()["pages"] and not b.has_work()


@pytest.mark.parametrize("name,dtype", [("B", "f32"), ("D", "bf16")])
def test_steps_with_prompt_portions_go_one_ahead_too(model_dirs, name, dtype):
    """Requests come while others decode, and their prompts are cut into portions: the step with the next portions
    and the others' next tokens is launched before the tokens of the step before it are read (a request that has
    just finished its prompt hands its first token on to its first decode step on the device).  Tokens, reasons
    and the cache's state are those of the engine that reads every step first; with penalties and stops too."""
    from inferrs_b200 import Engine
    cfg = CONFIG_B if name == "B" else __import__("helpers").CONFIG_D
    prompts = [random_tokens(n, cfg["vocab_size"], seed=60 + n) for n in (70, 9, 41, 26, 55, 3)]
    # in bfloat16 a row's rounding depends on which kernels the step's size selects: there all requests are
    # present from the start and none ends before the last prompt is in, so that both engines run the same steps
    late = dtype == "f32"
    kw = dict(dtype=dtype, block_size=16, num_blocks=64, max_batch_size=4 if late else 6, max_tokens_per_step=24,
              prefill_chunk=16)

    def run(overlap, params, late_every=3):
        eng = Engine(model_dirs[name], overlap=overlap, **kw)
        first = 2 if late else len(prompts)
        rids = [eng.add_request(p, q) for p, q in zip(prompts[:first], params[:first])]
        done, k, nxt = {}, 0, first
        while eng.has_work() or nxt < len(prompts):
            for r in eng.step():
                done[r.rid] = r
            k += 1
            if nxt < len(prompts) and k % late_every == 0:     # the next request arrives while the others run
                rids.append(eng.add_request(prompts[nxt], params[nxt]))
                nxt += 1
        for r in eng.flush():
            done[r.rid] = r
        assert eng.stats()["free_pages"] == eng.stats()["pages"] and not eng.has_work()
        eng.runner.manager.check_invariants()
        return [(done[r].output, done[r].finish_reason) for r in rids], eng

    greedy = [SamplingParams.greedy(max_tokens=16 + 4 * i) for i in range(len(prompts))]
    want, a = run(False, greedy)
    got, b = run(True, greedy)
    assert got == want
    assert b.stats()["portion_steps_ahead"] >= 8 and b.stats()["steps_ahead"] > b.stats()["portion_steps_ahead"]
    assert a.stats()["steps_ahead"] == 0
    # a stop token that the first request reaches while the later prompts are still coming in
    stop = want[0][0][6 if late else 15]
    stops = [SamplingParams(temperature=0.0, repetition_penalty=1.0, max_tokens=16 + 4 * i, stop_token_ids=(stop,))
             for i in range(len(prompts))]
    want, _ = run(False, stops)
    got, b = run(True, stops)
    assert got == want and any(reason == "stop" for _, reason in want)
    # the reference's default options (penalties over a window, top-k, top-p) with seeds
    sampled = [SamplingParams(temperature=0.7, max_tokens=16 + 2 * i, seed=5 + i) for i in range(len(prompts))]
    want, _ = run(False, sampled)
    got, b = run(True, sampled)
    assert got == want and b.stats()["portion_steps_ahead"] >= 8
