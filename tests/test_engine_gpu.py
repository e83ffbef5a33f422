"""The engine on the GPU against the plain implementation, in float32 and bfloat16: every way of
cutting requests into steps must give the same logits."""
import pytest
import torch

import plain_qwen3
from helpers import CONFIG_A, CONFIG_B, CONFIG_C, CONFIG_D, PAGE_SIZE, cut, random_tokens, rel_err
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.engine.loading import load_model_dir
from inferrs_b200.engine.runner import ModelRunner
from inferrs_b200.runtime import Runtime

pytestmark = pytest.mark.gpu

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}
# float32: 1e-4 against the plain implementation.  bfloat16: the plain implementation rounds where the engine stores
# bfloat16, so what is left is the order of sums and a few roundings that fall differently.
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}
_plain_cache = {}


def make_runner(model_dir, dtype, page_size, n_pages, max_requests=4):
    rt = Runtime.cuda(dtype)
    spec, weights, _ = load_model_dir(model_dir, rt)
    return ModelRunner(spec, weights, rt, page_size=page_size, n_pages=n_pages, max_requests=max_requests)


def plain_logits(model_dir, tokens, dtype):
    key = (model_dir, tuple(tokens), dtype)
    if key not in _plain_cache:
        cfg, w = plain_qwen3.read_model(model_dir)
        _plain_cache[key] = plain_qwen3.forward(cfg, w, tokens, store=None if dtype == torch.float32 else dtype)
    return _plain_cache[key]


def check(got, want, dtype, what=""):
    err = rel_err(got.cpu(), want)
    assert err < TOL[dtype], f"{what}: relative error {err:.3e}"
    if dtype == torch.float32:
        assert torch.equal(got.cpu().argmax(-1), want.argmax(-1)), f"{what}: greedy tokens differ"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole(model_dirs, name, dtype):
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=128)
    for i, n in enumerate([1, 5, 17, 33, 100]):
        toks = random_tokens(n, CONFIGS[name]["vocab_size"], seed=i)
        runner.admit(i)
        got = runner.step([StepEntry(i, toks, list(range(n)))])
        runner.release(i)
        check(got, plain_logits(model_dirs[name], toks, dtype), dtype, f"whole {n}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prefill_then_last_32_one_by_one(model_dirs, name, dtype):
    toks = random_tokens(150, CONFIGS[name]["vocab_size"], seed=11)
    want = plain_logits(model_dirs[name], toks, dtype)
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
    runner.admit("r")
    rows = [runner.step([StepEntry("r", toks[:118], list(range(118)))])]
    for t in range(118, 150):
        rows.append(runner.step([StepEntry("r", toks[t:t + 1], [0])]))
    check(torch.cat(rows), want, dtype, "decode after prefill")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(model_dirs, name, dtype):
    toks = random_tokens(131, CONFIGS[name]["vocab_size"], seed=12)
    want = plain_logits(model_dirs[name], toks, dtype)
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
    runner.admit("r")
    rows, at = [], 0
    for n in cut(len(toks), [7, 2, 13, 3, 2, 31, 1, 16]):
        rows.append(runner.step([StepEntry("r", toks[at:at + n], list(range(n)))]))
        at += n
    check(torch.cat(rows), want, dtype, "portions")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_requests_with_page_reuse(model_dirs, name, dtype):
    ps = PAGE_SIZE[name]
    lens = [70, 23, 97, 31, 18, 64, 5, 49]
    prompts = [random_tokens(n, CONFIGS[name]["vocab_size"], seed=20 + i) for i, n in enumerate(lens)]
    want = [plain_logits(model_dirs[name], p, dtype) for p in prompts]
    pages = lambda n: (n + ps - 1) // ps  # noqa: E731
    n_pages = pages(97) + pages(70) + pages(64) + pages(49) + 1  # too few for all: pages are used again
    runner = make_runner(model_dirs[name], dtype, ps, n_pages=n_pages)
    got = [[] for _ in prompts]
    at = [0] * len(prompts)
    live, nxt, step = [], 0, 0
    sizes = [5, 2, 9, 1, 3, 16, 1, 1, 27]
    while live or nxt < len(prompts):
        while len(live) < 4 and nxt < len(prompts) and \
                sum(pages(lens[i]) for i in live) + pages(lens[nxt]) <= n_pages:
            runner.admit(nxt)
            live.append(nxt)
            nxt += 1
        entries = []
        for k, i in enumerate(live):
            if (step + k) % 3 == 2 and len(live) > 1:
                continue
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
        check(torch.cat(got[i]), want[i], dtype, f"mixed request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_long_decode(model_dirs, name, dtype):
    toks = random_tokens(400, CONFIGS[name]["vocab_size"], seed=31)
    want = plain_logits(model_dirs[name], toks, dtype)
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=32)
    runner.admit("r")
    rows = [runner.step([StepEntry("r", toks[:3], [0, 1, 2])])]
    for t in range(3, 400):
        rows.append(runner.step([StepEntry("r", toks[t:t + 1], [0])]))
    check(torch.cat(rows), want, dtype, "long decode")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """From an empty cache, one token a step: position 0 alone, the first page while it fills, the first step over a
    page's edge; then a second request that starts beside the first one's decoding with portions of one, two and three
    tokens.  Every position against the plain implementation."""
    cfg = CONFIGS[name]
    n = 2 * PAGE_SIZE[name] + 3
    toks = random_tokens(n, cfg["vocab_size"], seed=61)
    other = random_tokens(6, cfg["vocab_size"], seed=62)
    want, want_other = plain_logits(model_dirs[name], toks, dtype), plain_logits(model_dirs[name], other, dtype)
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=8)
    runner.admit("r")
    rows, rows_other, at = [], [], 0
    for t in range(n):
        entries = [StepEntry("r", toks[t:t + 1], [0])]
        if t in (4, 5, 6):                                      # the other request's first tokens: 1, then 2, then 3
            if t == 4:
                runner.admit("o")
            k = t - 3
            entries.append(StepEntry("o", other[at:at + k], list(range(k))))
            at += k
        out = runner.step(entries)
        rows.append(out[:1])
        if len(entries) == 2:
            rows_other.append(out[1:])
    check(torch.cat(rows), want, dtype, "one token a step from an empty cache")
    check(torch.cat(rows_other), want_other, dtype, "a request that starts with portions of 1, 2 and 3 tokens")
    runner.release("r")
    runner.release("o")
    runner.manager.check_invariants()


@pytest.mark.parametrize("name,dtype", [("B", torch.float32), ("C", torch.bfloat16), ("D", torch.bfloat16),
                                        ("D", torch.float32)])
def test_steps_with_portions_are_replayed_graphs(model_dirs, name, dtype):
    """Steps with prompt portions are captured once per padded row count and replayed: the second request goes
    through replays only (other tokens, other pages, other lengths in the same shapes), two requests side by
    side share steps, and every logit still equals the plain implementation's."""
    cfg = CONFIGS[name]
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=96)
    pg = runner.portion_graphs
    assert pg is not None
    sizes = [40, 7, 2, 33, 90, 3, 1, 1, 25]
    n = sum(sizes)
    prompts = [random_tokens(n, cfg["vocab_size"], seed=60 + i) for i in range(4)]
    want = [plain_logits(model_dirs[name], p, dtype) for p in prompts]
    for i in (0, 1):
        runner.admit(i)
        rows, at = [], 0
        for s in sizes:
            w = list(range(max(0, s - 20), s))              # the last places of every portion
            rows.append((at + w[0], runner.step([StepEntry(i, prompts[i][at:at + s], w)])))
            at += s
        for first, out in rows:
            check(out, want[i][first:first + out.shape[0]], dtype, f"request {i} from {first}")
        if i == 0:
            captured = sorted(pg.captured)
            assert captured == [32, 64, 128], captured
    assert sorted(pg.captured) == captured, "the second request must not have needed a new capture"
    # two requests in the same steps, one a portion ahead of the other
    runner.admit(2)
    runner.admit(3)
    at = {2: 0, 3: 0}
    order = [(2, 0), (2, 1), (3, 0), (2, 2), (3, 1), (3, 2), (2, 3), (3, 3), (2, 4), (3, 4)]
    k = 0
    while k < len(order):
        entries, meta = [], []
        for rid, idx in order[k:k + 2]:
            if any(m[0] == rid for m in meta):
                break
            s = sizes[idx]
            w = [s - 1]
            entries.append(StepEntry(rid, prompts[rid][at[rid]:at[rid] + s], w))
            meta.append((rid, at[rid] + s - 1))
            at[rid] += s
        k += len(entries)
        out = runner.step(entries)
        for row, (rid, pos) in enumerate(meta):
            check(out[row:row + 1], want[rid][pos:pos + 1], dtype, f"request {rid} at {pos}")
    runner.manager.check_invariants()


@pytest.mark.parametrize("name,dtype", [("B", torch.float32), ("D", torch.bfloat16)])
def test_replayed_steps_take_tokens_that_are_still_on_the_device(model_dirs, name, dtype):
    """A step may name a token by its place in an int32 tensor on the device instead of by its id (the engine
    launches a step before it has read what the step before it sampled): a step of single tokens and a step
    with a portion beside single tokens, some tokens carried and some known, give the logits that the same step
    gives with all ids known; a step that is no replayed graph refuses."""
    cfg = CONFIGS[name]
    vocab = cfg["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=30 + n) for n in (21, 5, 34, 12)]
    nxt = [random_tokens(3, vocab, seed=70 + i) for i in range(4)]

    def play(carried):
        runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
        outs = []
        for i in (0, 1, 2):
            runner.admit(i)
            runner.step([StepEntry(i, prompts[i], [])])
        # the tokens of the next steps as an earlier step's output would hold them, in another order
        ids = torch.tensor([nxt[2][0], 0, nxt[0][0], nxt[1][0], nxt[0][1], nxt[2][1]], dtype=torch.int32, device="cuda")
        place = {(2, 0): 0, (0, 0): 2, (1, 0): 3, (0, 1): 4, (2, 1): 5}
        # three single tokens: request 1's is known, the others come from the device
        entries = [StepEntry(i, [nxt[i][0]], [0]) for i in (0, 1, 2)]
        if carried:
            entries = [StepEntry(0, [0], [0]), entries[1], StepEntry(2, [0], [0])]
            outs.append(runner.step(entries, carry=(ids, [place[(0, 0)], -1, place[(2, 0)]])))
        else:
            outs.append(runner.step(entries))
        # a new request's portion beside two single tokens, one of them carried
        runner.admit(3)
        entries = [StepEntry(0, [nxt[0][1]], [0]), StepEntry(3, prompts[3], [len(prompts[3]) - 1]),
                   StepEntry(2, [nxt[2][1]], [0])]
        if carried:
            entries[2] = StepEntry(2, [0], [0])
            outs.append(runner.step(entries, carry=(ids, [-1, -1, place[(2, 1)]])))
        else:
            outs.append(runner.step(entries))
        runner.manager.check_invariants()
        return outs, runner

    want, _ = play(False)
    got, runner = play(True)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    for i in (0, 2):
        full = plain_logits(model_dirs[name], prompts[i] + nxt[i][:2], dtype)
        check(got[0][i:i + 1], full[len(prompts[i]):len(prompts[i]) + 1], dtype, f"request {i}")
    with pytest.raises(ValueError, match="place"):
        runner.step([StepEntry(0, [0], [0])], carry=(torch.zeros(2, dtype=torch.int32, device="cuda"), [2]))
    with pytest.raises(ValueError, match="single token"):
        runner.step([StepEntry(1, [0, 0], [1])], carry=(torch.zeros(2, dtype=torch.int32, device="cuda"), [1]))
    runner.manager.check_invariants()
    plain_runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
    plain_runner.graphs = plain_runner.portion_graphs = None
    plain_runner.admit(0)
    with pytest.raises(ValueError, match="replayed"):
        plain_runner.step([StepEntry(0, [0], [0])], carry=(torch.zeros(1, dtype=torch.int32, device="cuda"), [0]))


def test_portions_through_the_kernel_with_two_query_tiles(tmp_path, monkeypatch):
    """The prefill attention kernel with two query tiles per CTA serves only large steps; here it is made to serve
    every step with a portion (head size 128, two query heads per key/value head, so a tile holds 2 x 64
    tokens): one request in portions that end inside the first query tile, inside the second and at their edges,
    then a request's portions beside decoded tokens of another, as replayed graphs; all logits against the plain
    implementation."""
    from inferrs_b200 import kernels
    from inferrs_b200.weights.random_init import write_random_model
    monkeypatch.setattr(kernels, "PAIR_MIN_CTAS", 1)
    calls = {"pair": 0}
    original = kernels.paged_attention_pair_tcgen05

    def counted(*a, **k):
        calls["pair"] += 1
        return original(*a, **k)

    monkeypatch.setattr(kernels, "paged_attention_pair_tcgen05", counted)
    cfg = dict(CONFIG_D, num_attention_heads=4, num_key_value_heads=2, hidden_size=160, intermediate_size=264)
    model_dir = str(tmp_path / "pair")
    write_random_model(model_dir, cfg, seed=11, dtype=torch.bfloat16)
    dtype = torch.bfloat16
    runner = make_runner(model_dir, dtype, 16, n_pages=96)
    sizes = [30, 64, 34, 128, 1, 65, 129, 3, 90]
    toks = [random_tokens(sum(sizes), cfg["vocab_size"], seed=70 + i) for i in range(3)]
    want = [plain_logits(model_dir, t, dtype) for t in toks]
    runner.admit(0)
    at = 0
    for s in sizes:
        out = runner.step([StepEntry(0, toks[0][at:at + s], list(range(s)))])
        check(out, want[0][at:at + s], dtype, f"portion of {s} from {at}")
        at += s
    assert calls["pair"] >= 4    # launched from Python where a step is not a replayed graph, and at every capture
    # a request's portions beside the decoded tokens of another, which has 100 tokens already
    runner.admit(1)
    runner.admit(2)
    runner.step([StepEntry(2, toks[2][:100], [])])
    at1, at2 = 0, 100
    for s in (50, 85, 7, 120):
        entries = [StepEntry(1, toks[1][at1:at1 + s], [s - 1]), StepEntry(2, toks[2][at2:at2 + 1], [0])]
        out = runner.step(entries)
        check(out[0:1], want[1][at1 + s - 1:at1 + s], dtype, f"request 1 at {at1 + s - 1}")
        check(out[1:2], want[2][at2:at2 + 1], dtype, f"request 2 at {at2}")
        at1 += s
        at2 += 1
    assert kernels.attention_pair_tcgen05_error() == 0
    runner.manager.check_invariants()


@pytest.mark.parametrize("name", ["D", "B"])
def test_a_replayed_step_of_portions_alone_gives_what_the_plain_step_gives_every_time(model_dirs, name):
    """A captured step that holds prompt portions only launches the kernel for single tokens with nothing to do.
    Its kernels start before their predecessors have ended (programmatic dependent launch), so a kernel that left
    without waiting would let its successor read queries and keys that are not written yet.  The same captured
    step is replayed many times with other tokens; every replay must give what the step launched plainly gives
    (the same bits in float32; in bfloat16 the library may multiply 100 rows another way than the padded 128)."""
    dtype = torch.bfloat16 if name == "D" else torch.float32
    cfg = CONFIGS[name]
    plain = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
    plain.graphs = plain.portion_graphs = None
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=64)
    assert runner.portion_graphs is not None
    n, want_rows = 100, list(range(60, 100))
    for i in range(40):
        toks = random_tokens(n, cfg["vocab_size"], seed=900 + i)
        plain.admit(i)
        want = plain.step([StepEntry(i, toks, want_rows)])
        plain.release(i)
        runner.admit(i)
        got = runner.step([StepEntry(i, toks, want_rows)])
        runner.release(i)
        if dtype == torch.float32:
            assert torch.equal(got, want), f"replay {i}"
        else:
            assert rel_err(got, want) < 1e-2, f"replay {i}"
    assert sorted(runner.portion_graphs.captured) == [128]
    check(got, plain_logits(model_dirs[name], toks, dtype)[60:], dtype, "the last replay")


def test_the_positions_of_the_published_checkpoints(tmp_path):
    """max_position_embeddings as large as the published checkpoints' (40,960): the rotation tables, the block
    tables of replayed steps (2,560 pages wide) and their descriptions have that size; a request far beyond the
    sizes of the other tests is decoded and compared with the plain implementation."""
    from inferrs_b200.weights.random_init import write_random_model
    cfg = dict(CONFIG_D, max_position_embeddings=40960)
    model_dir = str(tmp_path / "wide")
    write_random_model(model_dir, cfg, seed=21, dtype=torch.bfloat16)
    dtype = torch.bfloat16
    runner = make_runner(model_dir, dtype, 16, n_pages=2600, max_requests=2)
    assert runner.graphs.fixed_pages == [2560] and runner.graphs.max_context == 40960
    n_prompt, n_decode = 2500, 24
    toks = random_tokens(n_prompt + n_decode, cfg["vocab_size"], seed=5)
    want = plain_logits(model_dir, toks, dtype)
    runner.admit("r")
    at, rows = 0, []
    for n in (1000, 1000, 500):          # replayed steps of 1,024 and 512 rows
        out = runner.step([StepEntry("r", toks[at:at + n], [n - 1])])
        check(out, want[at + n - 1:at + n], dtype, f"the portion that ends at {at + n}")
        at += n
    for t in range(n_prompt, n_prompt + n_decode):
        rows.append(runner.step([StepEntry("r", toks[t:t + 1], [0])]))
    check(torch.cat(rows), want[n_prompt:], dtype, "decoding at 2,500 tokens with block tables of 2,560 pages")
    assert sorted(runner.graphs.captured) == [1] and sorted(runner.portion_graphs.captured) == [512, 1024]


def test_decode_steps_fold_the_norms_into_the_products(model_dirs, monkeypatch):
    """In a step of a few rows the addition to the residual stream and the norm between two products run inside the
    products (head size 128, bfloat16): the norm kernel is then launched for the first layer's first norm and the last
    norm only, and the logits are those of the same step with every norm as a kernel of its own."""
    from inferrs_b200 import kernels
    name, dtype = "D", torch.bfloat16
    toks = random_tokens(60, CONFIGS[name]["vocab_size"], seed=77)
    want = plain_logits(model_dirs[name], toks, dtype)

    def decode(fold):
        if not fold:
            monkeypatch.setattr(kernels, "folded_norm_supported", lambda *a, **k: False)
        calls = {"n": 0}
        original = kernels.add_rms_norm

        def counted(*a, **k):
            calls["n"] += 1
            return original(*a, **k)

        monkeypatch.setattr(kernels, "add_rms_norm", counted)
        runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=16)
        runner.graphs = runner.portion_graphs = None          # launched one by one, so that the launches can be counted
        runner.admit("r")
        runner.step([StepEntry("r", toks[:40], [])])
        calls["n"] = 0
        rows = [runner.step([StepEntry("r", toks[t:t + 1], [0])]) for t in range(40, 60)]
        monkeypatch.undo()
        return torch.cat(rows), calls["n"] / 20

    folded, n_folded = decode(True)
    plain, n_plain = decode(False)
    layers = CONFIGS[name]["num_hidden_layers"]
    assert n_plain == 2 * layers + 1 and n_folded == 2, (n_plain, n_folded)
    check(folded, want[40:], dtype, "folded norms")
    check(plain, want[40:], dtype, "norm kernels")
    assert rel_err(folded, plain) < 2e-2


def test_steps_of_many_short_prompts_take_the_longer_tile_list(model_dirs):
    """A captured step with prompt portions exists for up to eight requests that bring attention tiles and for as many
    as the cache admits: twelve short prompts in one step, beside a longer one and a decoding request, are replayed by
    the second and give what the plain implementation gives; a step of three prompts afterwards takes the first."""
    name, dtype = "B", torch.float32
    cfg = CONFIGS[name]
    runner = make_runner(model_dirs[name], dtype, PAGE_SIZE[name], n_pages=96, max_requests=16)
    pg = runner.portion_graphs
    assert pg is not None and pg.tile_pads == [8, 17]
    lens = [5, 2, 9, 3, 17, 2, 6, 4, 11, 2, 7, 3]
    prompts = [random_tokens(n, cfg["vocab_size"], seed=300 + i) for i, n in enumerate(lens)]
    long_one = random_tokens(40, cfg["vocab_size"], seed=299)
    decoding = random_tokens(21, cfg["vocab_size"], seed=298)
    runner.admit("d")
    runner.step([StepEntry("d", decoding[:20], [])])
    entries = [StepEntry("d", decoding[20:], [0]), StepEntry("long", long_one, [39])]
    entries += [StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)]
    for e in entries[1:]:
        runner.admit(e.rid)
    out = runner.step(entries)
    rows = sum(len(e.tokens) for e in entries)
    bucket = pg.bucket_for(rows)
    assert sorted(pg.captured[bucket]) == [17], "thirteen requests bring tiles: the list for eight does not hold them"
    check(out[0:1], plain_logits(model_dirs[name], decoding, dtype)[20:], dtype, "the decoding request")
    check(out[1:2], plain_logits(model_dirs[name], long_one, dtype)[39:], dtype, "the longer prompt")
    for i, p in enumerate(prompts):
        check(out[2 + i:3 + i], plain_logits(model_dirs[name], p, dtype)[-1:], dtype, f"short prompt {i}")
    for e in entries:
        runner.release(e.rid)
    few = [random_tokens(n, cfg["vocab_size"], seed=400 + n) for n in (30, 41, 37)]
    for i, p in enumerate(few):
        runner.admit(("few", i))
    out = runner.step([StepEntry(("few", i), p, [len(p) - 1]) for i, p in enumerate(few)])
    assert bucket == pg.bucket_for(sum(map(len, few))) and sorted(pg.captured[bucket]) == [8, 17]
    for i, p in enumerate(few):
        check(out[i:i + 1], plain_logits(model_dirs[name], p, dtype)[-1:], dtype, f"one of three prompts, {i}")
        runner.release(("few", i))
    runner.manager.check_invariants()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,width,inner,vocab,page", [
    (5, 5, 48, 88, 120, 263, 8), (7, 1, 80, 136, 72, 149, 16), (9, 3, 112, 104, 152, 211, 4), (3, 1, 144, 56, 200, 331, 16),
    (2, 2, 256, 72, 88, 97, 16), (12, 4, 96, 200, 136, 401, 8)])
def test_head_sizes_in_steps_of_sixteen_and_odd_numbers_of_heads(tmp_path, dtype, heads, kv_heads, head_dim, width, inner,
                                                                 vocab, page):
    """Sizes that no kernel written for head size 64, 128 or 256 and groups of a power of two takes for granted: the
    dispatch has to find a kernel for each or say clearly that there is none; what runs must agree with the plain
    implementation, whole and cut into portions and single tokens beside another request."""
    from inferrs_b200.weights.random_init import write_random_model
    cfg = dict(CONFIG_A, num_hidden_layers=2, hidden_size=width, num_attention_heads=heads, num_key_value_heads=kv_heads,
               head_dim=head_dim, intermediate_size=inner, vocab_size=vocab, rms_norm_eps=3e-6, rope_theta=30000.0)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=heads * 100 + head_dim, dtype=torch.bfloat16)
    toks = random_tokens(70, vocab, seed=head_dim)
    other = random_tokens(23, vocab, seed=head_dim + 1)
    want, want_other = plain_logits(folder, toks, dtype), plain_logits(folder, other, dtype)
    runner = make_runner(folder, dtype, page, n_pages=(70 + 23) // page + 6)
    runner.admit("w")
    check(runner.step([StepEntry("w", toks, list(range(70)))]), want, dtype, "whole")
    runner.release("w")
    runner.admit("a")
    runner.admit("b")
    rows_a, rows_b, at, bt = [], [], 0, 0
    for n, m in ((9, 0), (2, 11), (31, 1), (1, 1), (1, 7), (17, 1), (1, 2), (8, 0)):
        entries = [StepEntry("a", toks[at:at + n], list(range(n)))]
        if m:
            entries.append(StepEntry("b", other[bt:bt + m], list(range(m))))
        out = runner.step(entries)
        rows_a.append(out[:n])
        if m:
            rows_b.append(out[n:])
        at, bt = at + n, bt + m
    assert at == 70 and bt == 23
    check(torch.cat(rows_a), want, dtype, "portions and single tokens")
    check(torch.cat(rows_b), want_other, dtype, "the request beside it")
    runner.release("a")
    runner.release("b")
    runner.manager.check_invariants()
