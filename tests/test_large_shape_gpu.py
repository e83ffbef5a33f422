"""The layer sizes of Qwen3-8B (two layers of them, the whole vocabulary) against the plain implementation,
in float32 and in bfloat16, in the four ways of cutting requests into steps.  At these sizes the bfloat16 run
goes through the kernels that serving uses: the tcgen05 products for few rows and the library's for many, the
gated product, the TMA decode attention and the tcgen05 prefill attention."""
import pytest
import torch

import plain_qwen3
from helpers import cut, random_tokens, rel_err
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.engine.loading import random_model
from inferrs_b200.engine.runner import ModelRunner
from inferrs_b200.runtime import Runtime

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 4096, "tie_word_embeddings": False, "hidden_act": "silu",
}
N_TOKENS = 88
LAST = 32
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}


@pytest.fixture(scope="module", params=[torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def setup(request):
    dtype = request.param
    rt = Runtime.cuda(dtype)
    spec, weights, _ = random_model(CONFIG, 5, rt)
    host = {k: v.float().cpu() for k, v in weights.items()}
    prompts = [random_tokens(N_TOKENS, CONFIG["vocab_size"], seed=20 + i) for i in range(2)]
    store = None if dtype == torch.float32 else dtype
    want = [plain_qwen3.forward(CONFIG, host, p, store=store)[-LAST:] for p in prompts]
    del host
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=14, max_requests=4)
    yield dtype, runner, prompts, want
    del runner, weights
    torch.cuda.empty_cache()


def check(got, want, dtype, what):
    err = rel_err(got.cpu(), want)
    assert err < TOL[dtype], f"{what}: relative error {err:.3e}"
    if dtype == torch.float32:
        assert torch.equal(got.cpu().argmax(-1), want.argmax(-1)), f"{what}: greedy tokens differ"


def run_cut(runner, rid, toks, sizes):
    """The logits of the last LAST tokens of a request fed in portions of the given sizes."""
    runner.admit(rid)
    rows, at = [], 0
    for n in sizes:
        want = [i for i in range(n) if at + i >= len(toks) - LAST]
        out = runner.step([StepEntry(rid, toks[at:at + n], want)])
        if want:
            rows.append(out)
        at += n
    runner.release(rid)
    return torch.cat(rows)


def test_whole(setup):
    dtype, runner, prompts, want = setup
    check(run_cut(runner, "w", prompts[0], [N_TOKENS]), want[0], dtype, "whole")


def test_most_in_one_step_then_one_by_one(setup):
    dtype, runner, prompts, want = setup
    check(run_cut(runner, "d", prompts[0], [N_TOKENS - LAST] + [1] * LAST), want[0], dtype, "decoded")


def test_portions_of_changing_size(setup):
    dtype, runner, prompts, want = setup
    check(run_cut(runner, "p", prompts[1], cut(N_TOKENS, [7, 2, 13, 3, 2, 30])), want[1], dtype, "portions")


def test_mixed_with_pages_used_again(setup):
    """Both requests live at once, portions of one beside decoded tokens of the other, in a pool of 14 pages
    (two requests of 88 tokens need 12) after the tests above have used and given back every page."""
    dtype, runner, prompts, want = setup
    a, b = prompts
    runner.admit("a")
    runner.admit("b")
    got = {"a": [], "b": []}
    at = {"a": 0, "b": 0}

    def entry(rid, toks, n):
        w = [i for i in range(n) if at[rid] + i >= N_TOKENS - LAST]
        e = StepEntry(rid, toks[at[rid]:at[rid] + n], w)
        at[rid] += n
        return e, bool(w)

    plan = [(40, 0), (16, 30), (1, 11), (1, 2), (1, 13)] + [(1, 1)] * 29 + [(0, 1)] * 3
    for na, nb in plan:
        entries, keep = [], []
        for rid, toks, n in (("a", a, na), ("b", b, nb)):
            n = min(n, N_TOKENS - at[rid])
            if n > 0:
                e, has = entry(rid, toks, n)
                entries.append(e)
                keep.append((rid, len(e.want)))
        if not entries:
            continue
        out = runner.step(entries)
        row = 0
        for rid, k in keep:
            if k:
                got[rid].append(out[row:row + k])
                row += k
    assert at == {"a": N_TOKENS, "b": N_TOKENS}
    check(torch.cat(got["a"]), want[0], dtype, "mixed a")
    check(torch.cat(got["b"]), want[1], dtype, "mixed b")
    runner.release("a")
    runner.release("b")
    runner.manager.check_invariants()


# ---- the sizes that the measured steps have: a prompt of 2,048 tokens in one step, portions of 512 beside a
# decoding request, decoding at more than 2,048 tokens -------------------------------------------------------
LONG, LONG_DECODE = 2048, 40
MID, MID_DECODE = 1100, 8


@pytest.fixture(scope="module", params=[torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def long_setup(request):
    dtype = request.param
    rt = Runtime.cuda(dtype)
    spec, weights, _ = random_model(CONFIG, 6, rt)
    host = {k: v.float().cpu() for k, v in weights.items()}
    long_toks = random_tokens(LONG + LONG_DECODE, CONFIG["vocab_size"], seed=40)
    mid_toks = random_tokens(MID + MID_DECODE, CONFIG["vocab_size"], seed=41)
    store = None if dtype == torch.float32 else dtype
    want_long = plain_qwen3.forward(CONFIG, host, long_toks, store=store, last=LAST + LONG_DECODE)
    want_mid = plain_qwen3.forward(CONFIG, host, mid_toks, store=store, last=LAST + MID_DECODE)
    del host
    pages = (LONG + LONG_DECODE + 15) // 16 + (MID + MID_DECODE + 15) // 16 + 2
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=pages, max_requests=4)
    yield dtype, runner, long_toks, mid_toks, want_long, want_mid
    del runner, weights
    torch.cuda.empty_cache()


def test_the_steps_that_are_measured(long_setup):
    """A prompt of 2,048 tokens as one step (in bfloat16: a replayed graph of 2,048 rows, the library's products,
    the rotation kernel for many rows, the attention kernel with two query tiles); then a second request's prompt
    of 1,100 tokens in portions of 512 beside the first request's decoded tokens; then both decode, the first at
    more than 2,048 tokens (its keys in several slices)."""
    from inferrs_b200 import kernels
    dtype, runner, long_toks, mid_toks, want_long, want_mid = long_setup
    pair_calls = {"n": 0}
    original = kernels.paged_attention_pair_tcgen05

    def counted(*a, **k):
        pair_calls["n"] += 1
        return original(*a, **k)

    kernels.paged_attention_pair_tcgen05 = counted
    try:
        runner.admit("long")
        got_long = [runner.step([StepEntry("long", long_toks[:LONG], list(range(LONG - LAST, LONG)))])]
    finally:
        kernels.paged_attention_pair_tcgen05 = original
    if dtype == torch.bfloat16:
        assert pair_calls["n"] > 0, "a step of 2,048 rows was meant to run the kernel with two query tiles"
        assert 2048 in runner.portion_graphs.captured
    check(got_long[0], want_long[:LAST], dtype, "the prompt of 2,048 tokens in one step")
    runner.admit("mid")
    got_mid, at_long, at_mid = [], LONG, 0
    for n in (512, 512, MID - 1024):
        w = [i for i in range(n) if at_mid + i >= MID - LAST]
        out = runner.step([StepEntry("long", long_toks[at_long:at_long + 1], [0]),
                           StepEntry("mid", mid_toks[at_mid:at_mid + n], w)])
        got_long.append(out[:1])
        if w:
            got_mid.append(out[1:])
        at_long += 1
        at_mid += n
    while at_long < LONG + LONG_DECODE:
        entries = [StepEntry("long", long_toks[at_long:at_long + 1], [0])]
        if at_mid < MID + MID_DECODE:
            entries.append(StepEntry("mid", mid_toks[at_mid:at_mid + 1], [0]))
        out = runner.step(entries)
        got_long.append(out[:1])
        if len(entries) == 2:
            got_mid.append(out[1:])
            at_mid += 1
        at_long += 1
    assert at_mid == MID + MID_DECODE
    check(torch.cat(got_long), want_long, dtype, "the long request: last 32 places of its prompt, then decoded")
    check(torch.cat(got_mid), want_mid, dtype, "the second request: portions of 512 beside decoded tokens")
    if dtype == torch.bfloat16:
        assert kernels.attention_pair_tcgen05_error() == 0 and kernels.attention_tcgen05_error() == 0
        assert kernels.attention_decode_error() == 0 and kernels.gemm_tcgen05_error() == 0
    runner.release("long")
    runner.release("mid")
    runner.manager.check_invariants()


# ---- the layer sizes of the other two checkpoints that are measured: Qwen3-0.6B (a narrow stream, two query heads per
# key/value head, tied embeddings) and Qwen3-32B (eight query heads per key/value head, a wide feed-forward) ----------
OTHER_SHAPES = {
    "0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                 tie_word_embeddings=True, num_hidden_layers=2),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600,
                tie_word_embeddings=False, num_hidden_layers=1),
}


@pytest.mark.parametrize("shape", sorted(OTHER_SHAPES))
def test_the_other_checkpoints_layer_sizes(shape):
    """bfloat16, the whole vocabulary: a prompt of 300 tokens in two portions (the second beside another request's
    first), then both requests decode eight tokens side by side; the last 32 places of the first prompt and every
    decoded place against the plain implementation."""
    dtype = torch.bfloat16
    config = dict(CONFIG, **OTHER_SHAPES[shape])
    rt = Runtime.cuda(dtype)
    spec, weights, _ = random_model(config, 9, rt)
    host = {k: v.float().cpu() for k, v in weights.items()}
    n_a, n_b, n_dec = 300, 70, 8
    a = random_tokens(n_a + n_dec, config["vocab_size"], seed=50)
    b = random_tokens(n_b + n_dec, config["vocab_size"], seed=51)
    want_a = plain_qwen3.forward(config, host, a, store=dtype, last=LAST + n_dec)
    want_b = plain_qwen3.forward(config, host, b, store=dtype, last=n_dec + 1)
    del host
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=(n_a + n_b + 2 * n_dec) // 16 + 4, max_requests=4)
    runner.admit("a")
    runner.admit("b")
    runner.step([StepEntry("a", a[:200], [])])
    got_a = []
    out = runner.step([StepEntry("a", a[200:n_a], list(range(n_a - 200 - LAST, n_a - 200))),
                       StepEntry("b", b[:n_b], [n_b - 1])])
    got_a.append(out[:LAST])
    got_b = [out[LAST:]]
    for i in range(n_dec):
        out = runner.step([StepEntry("a", a[n_a + i:n_a + i + 1], [0]), StepEntry("b", b[n_b + i:n_b + i + 1], [0])])
        got_a.append(out[:1])
        got_b.append(out[1:])
    check(torch.cat(got_a), want_a, dtype, f"{shape}: the first request")
    check(torch.cat(got_b), want_b, dtype, f"{shape}: the second request")
    from inferrs_b200 import kernels
    assert kernels.attention_decode_error() == 0 and kernels.gemm_tcgen05_error() == 0
    assert kernels.attention_tcgen05_error() == 0 and kernels.attention_pair_tcgen05_error() == 0
    runner.release("a")
    runner.release("b")
    runner.manager.check_invariants()
    del runner, weights
    torch.cuda.empty_cache()
