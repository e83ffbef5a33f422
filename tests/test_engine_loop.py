"""The engine's loop with steps launched one ahead, on the CPU: a stand-in for the model (a rolling hash of the
tokens it is fed) and for the sampler (the next token is a function of that hash) under the real scheduler and
cache book.  What the loop may get wrong shows in the tokens: a token taken from the wrong place of the step
before, a step planned from a stale count, a request that is fed a token twice or not at all."""
import random

import pytest
import torch

from inferrs_b200.cache.manager import CacheManager, GroupLayout
from inferrs_b200.engine.engine import Engine
from inferrs_b200.engine.scheduler import Scheduler
from inferrs_b200.sampling.params import SamplingParams

VOCAB = 50
MOD = 1_000_003


def next_token(h: int) -> int:
    return (h * 7919 + 13) % VOCAB


class FakeRunner:
    """Feeds every token it is given into its request's hash; the "logits" of a wanted place are the hash there.
    Knows a preempted request by its empty cache and starts its hash anew."""
    graphs = object()            # the engine asks only whether there are replayed graphs at all

    def __init__(self, manager, carries_up_to_rows):
        self.manager = manager
        self.hash = {}
        self.carries_up_to_rows = carries_up_to_rows
        self.n_carried = 0

    def takes_carried_tokens(self, entries):
        return sum(len(e.tokens) for e in entries) <= self.carries_up_to_rows

    def step(self, entries, own_output=True, carry=None):
        self.manager.reserve({e.rid: len(e.tokens) for e in entries})
        out = []
        for k, e in enumerate(entries):
            toks = list(e.tokens)
            if carry is not None and carry[1][k] >= 0:
                assert len(toks) == 1 and self.takes_carried_tokens(entries)
                toks = [int(carry[0][carry[1][k]])]
                self.n_carried += 1
            h = 0 if self.manager.n_tokens(e.rid) == 0 else self.hash[e.rid]
            for i, t in enumerate(toks):
                h = (h * 31 + t + 7) % MOD
                if i in e.want:
                    out.append(h)
            self.hash[e.rid] = h
            self.manager.commit(e.rid, len(toks))
        return torch.tensor(out, dtype=torch.int64)


class FakeSampler:
    def sample(self, logits, params, seeds, histories, pending=0, pending_ids=None, pending_from=None):
        return torch.tensor([next_token(int(h)) for h in logits], dtype=torch.int32)


def plain_generate(prompt, params, eos):
    h, out = 0, []
    for t in prompt:
        h = (h * 31 + t + 7) % MOD
    while True:
        tok = next_token(h)
        out.append(tok)
        if not params.ignore_eos and (tok in eos or tok in params.stop_token_ids):
            return out, "stop"
        if len(out) >= params.max_tokens:
            return out, "length"
        h = (h * 31 + tok + 7) % MOD


def make_engine(overlap, n_pages, page_size, slots, max_batch, budget, chunk, eos, carries_up_to_rows=10 ** 9):
    eng = Engine.__new__(Engine)                 # the loop alone: no model is loaded, no device is touched
    manager = CacheManager([GroupLayout("full")], page_size, [n_pages], slots)
    eng.rt = type("Rt", (), {"device": torch.device("cpu"), "dtype": torch.float32})()
    eng.spec = type("Spec", (), {"vocab_size": VOCAB})()
    eng.runner = FakeRunner(manager, carries_up_to_rows)
    eng.scheduler = Scheduler(manager, max_batch, budget, 10_000, eos, chunk)
    eng.sampler = FakeSampler()
    eng.max_seq_len = 10_000
    eng._ids = iter(range(10 ** 9))
    eng._rng = random.Random(0)
    eng.n_steps = eng.n_tokens_run = eng.n_steps_in_vain = eng.n_steps_ahead = eng.n_portion_steps_ahead = 0
    eng.overlap = overlap
    eng._in_flight = None
    eng._pinned = []
    eng.health = None
    eng.kernel_errors, eng._unchecked, eng._checked_up_to, eng._last_look = [], [], 0, 0
    return eng, manager


@pytest.mark.parametrize("seed", range(8))
def test_steps_one_ahead_give_what_the_plain_loop_gives(seed):
    """Random prompts, token limits, stop tokens and arrival times; a cache so small that requests are preempted;
    an abort; steps that cannot take tokens from the device (too many rows for the stand-in's "graphs").  With
    and without steps launched ahead every request must end with the tokens and the reason of the plain loop."""
    rng = random.Random(seed)
    eos = (3,)
    page_size, n_pages, slots = rng.choice([(4, 40, 6), (8, 16, 4), (4, 64, 8)])
    max_batch, budget, chunk = rng.choice([(4, 24, 8), (6, 16, None), (3, 12, 5)])
    carries = rng.choice([10 ** 9, 10 ** 9, 9])
    requests = []
    for i in range(14):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.choice([1, 3, 8, 15, 30, 47]))]
        params = SamplingParams(temperature=0.0, repetition_penalty=1.0, max_tokens=rng.choice([1, 2, 7, 20, 33]),
                                stop_token_ids=rng.choice([(), (5,), (5, 11, 17)]), ignore_eos=rng.random() < 0.25)
        requests.append((rng.randrange(0, 40), prompt, params))
    aborted = rng.randrange(len(requests))
    abort_at = rng.randrange(5, 60)
    results = {}
    for overlap in (False, True):
        eng, manager = make_engine(overlap, n_pages, page_size, slots, max_batch, budget, chunk, eos, carries)
        done, turn, live = {}, 0, {}
        while turn < 2000 and (eng.has_work() or len(live) < len(requests)):
            for i, (arrives, prompt, params) in enumerate(requests):
                if arrives == turn:
                    live[i] = eng.add_request(prompt, params, rid=i)
            if turn == abort_at and aborted in live and aborted not in done:
                r = eng.abort(aborted)
                if r is not None:
                    done[aborted] = r
            for r in eng.step():
                done[r.rid] = r
            manager.check_invariants()
            eng.scheduler.check()
            turn += 1
        for r in eng.flush():
            done[r.rid] = r
        assert sorted(done) == list(range(len(requests))) and not eng.has_work()
        assert manager.pools[0].n_free == n_pages and manager.n_live == 0
        results[overlap] = ({i: (r.output, r.finish_reason) for i, r in done.items()}, eng)
    for i, (_, prompt, params) in enumerate(requests):
        for overlap in (False, True):
            output, reason = results[overlap][0][i]
            if reason == "cancelled":
                assert i == aborted
                want, _ = plain_generate(prompt, params, eos)
                assert output == want[:len(output)]
            else:
                assert (output, reason) == plain_generate(prompt, params, eos), (i, overlap)
    ahead = results[True][1]
    assert ahead.n_steps_ahead > 10 and ahead.runner.n_carried > 10
    assert results[False][1].n_steps_ahead == 0 and results[False][1].runner.n_carried == 0


def test_carried_tokens_are_named_in_the_description():
    """In a step's description the token ids come first, in the order of the entries; an entry whose token is still
    on the device gets -1 - place there, and only an entry of one token may have a place."""
    from inferrs_b200.engine.batch import StepEntry
    from inferrs_b200.engine.graphs import name_carried_tokens
    stage = torch.arange(100, 120, dtype=torch.int32)
    entries = [StepEntry("a", [7], [0]), StepEntry("b", [1, 2, 3], []), StepEntry("c", [9], [0]), StepEntry("d", [4], [0])]
    rows = name_carried_tokens(stage, entries, [2, -1, -1, 0])
    assert rows == 6
    assert stage.tolist()[:8] == [-3, 101, 102, 103, 104, -1, 106, 107]
    with pytest.raises(ValueError, match="single token"):
        name_carried_tokens(stage, entries, [-1, 1, -1, -1])


class FakeHealth:
    """Stands in for the reader of the kernels' error words: the look asked for as the ``fail_at``-th one finds a word
    set, the others find nothing; an answer arrives one poll after it was asked for."""

    def __init__(self, fail_at, every=4):
        self.every, self.fail_at = every, fail_at
        self.asked, self.age, self.n_reset, self.pending = 0, 0, 0, False

    def queue(self):
        assert not self.pending
        self.pending, self.age = True, 0
        self.asked += 1

    def poll(self, wait=False):
        if not self.pending:
            return None
        self.age += 1
        if not wait and self.age < 2:
            return None
        self.pending = False
        return {"decode attention": 2} if self.asked == self.fail_at else {}

    def reset(self):
        self.n_reset += 1
        return {}


@pytest.mark.parametrize("overlap", [False, True])
def test_a_word_that_a_kernel_set_ends_the_requests_that_it_may_have_touched(overlap):
    """The engine asks for the kernels' error words every few steps and when a request ends, and reads the answer
    when it is there.  When a word is set, the running requests and those that ended since the last look that found
    nothing end with "error", the words are cleared, every page comes back, and the waiting requests run as if
    nothing had happened."""
    eos = ()
    eng, manager = make_engine(overlap, n_pages=64, page_size=4, slots=3, max_batch=3, budget=16, chunk=None, eos=eos)
    eng.health = FakeHealth(fail_at=4)
    params = [SamplingParams(temperature=0.0, max_tokens=n) for n in (3, 40, 40, 9, 12, 5)]
    prompts = [[(7 * i + j) % VOCAB for j in range(5 + i)] for i in range(len(params))]
    for i, (p, sp) in enumerate(zip(prompts, params)):
        eng.add_request(p, sp, rid=i)
    done, turns = {}, 0
    while eng.has_work() and turns < 500:
        for r in eng.step():
            done[r.rid] = r
        manager.check_invariants()
        turns += 1
    for r in eng.flush():
        done[r.rid] = r
    assert sorted(done) == list(range(len(params)))
    assert eng.health.n_reset == 1 and len(eng.kernel_errors) == 1
    assert eng.kernel_errors[0]["words"] == {"decode attention": 2}
    failed = sorted(i for i, r in done.items() if r.finish_reason == "error")
    assert 1 in failed and 2 in failed, "the requests that were running when the word was found"
    assert len(failed) < len(params), "requests that came after the words were cleared must run"
    for i, r in done.items():
        if r.finish_reason != "error":
            assert (r.output, r.finish_reason) == plain_generate(prompts[i], params[i], eos), i
        else:
            want, _ = plain_generate(prompts[i], params[i], eos)
            assert r.output == want[:len(r.output)]
    assert manager.pools[0].n_free == 64 and manager.n_live == 0
