"""The Python entry point: ``Engine(model_dir).generate(prompts, sampling)``.

Token ids in, token ids out.  The engine puts together what the reference's ``load_engine`` and
``Engine::run`` do (inferrs/src/engine.rs:104-207, :1366-1912): load the model named by config.json,
size and attach the paged cache, then loop: plan a step, run it, sample, finish and free.
Option names follow the reference's command line (inferrs/src/main.rs:91-204).
"""
from __future__ import annotations

import itertools
import random
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.base import generation_eos_ids
from ..runtime import Runtime, parse_dtype
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .health import KernelHealth
from .loading import load_model_dir, random_model
from .runner import ModelRunner
from .scheduler import PlannedEntry, Request, Scheduler


class KernelFault(RuntimeError):
    """A kernel reported that it could not do its work (see :mod:`inferrs_b200.engine.health`)."""


class Engine:
    """
    model_dir            folder with config.json and model.safetensors (or shards)
    dtype                "bf16" (default) or "f32"
    block_size           tokens per cache page (reference: --block-size, 16)
    num_blocks           pages in the cache; None: sized from ``paged_attention``
    paged_attention      fraction of the device's free memory, after the weights, given to the cache
                         (reference: --paged-attention[=0.9] is a fraction of total memory)
    max_batch_size       most requests in a step (reference: --max-batch-size, 32)
    max_tokens_per_step  token budget of a step (reference: --max-tokens-per-step, 2048)
    max_seq_len          0: the model's max_position_embeddings (reference: --max-seq-len)
    config, random_weights   instead of ``model_dir``: a config.json dictionary and a seed; the weights
                         are made on the device
    overlap              steps are launched one ahead: while the device runs a step, the host plans and launches
                         the next one (a token that the running step samples is handed on to it on the device)
                         and only then reads the running step's tokens; a request that turns out to have ended
                         runs one step in vain.  Results are the same; ``step`` then reports a request's end one
                         call later.  Where the next step needs a running request's pages, ends a request for
                         sure or is no replayed graph, the tokens are read first.
    """

    def __init__(self, model_dir: Optional[str] = None, dtype: str = "bf16", block_size: int = 16,
                 num_blocks: Optional[int] = None, paged_attention: float = 0.9, max_batch_size: int = 32,
                 max_tokens_per_step: int = 2048, max_seq_len: int = 0, prefill_chunk: Optional[int] = None,
                 config: Optional[dict] = None, random_weights: Optional[int] = None,
                 runtime: Optional[Runtime] = None, overlap: bool = True):
        self.rt = runtime if runtime is not None else Runtime.cuda(parse_dtype(dtype))
        if model_dir is not None:
            spec, weights, cfg = load_model_dir(model_dir, self.rt)
        elif config is not None and random_weights is not None:
            spec, weights, cfg = random_model(config, random_weights, self.rt)
        else:
            raise ValueError("give a model_dir, or a config dictionary with a random_weights seed")
        self.spec, self.config = spec, cfg
        # what ends a request by itself: config.json's ids and, from a model folder, generation_config.json's
        eos = tuple(spec.eos_token_ids)
        if model_dir is not None:
            eos += tuple(t for t in generation_eos_ids(model_dir, spec.vocab_size) if t not in eos)
        self.eos_token_ids = eos
        self.max_seq_len = min(max_seq_len, spec.max_positions) if max_seq_len else spec.max_positions
        # the cache is sized (num_blocks None) once the model stands and the tensors that were fused into others
        # have been given back: only then does the free memory say what is left
        self.runner = ModelRunner(spec, weights, self.rt, page_size=block_size, n_pages=num_blocks,
                                  max_requests=max_batch_size, max_context=self.max_seq_len,
                                  cache_fraction=paged_attention, consume_weights=True)
        del weights
        self.scheduler = Scheduler(self.runner.manager, max_batch_size, max_tokens_per_step, self.max_seq_len,
                                   self.eos_token_ids, prefill_chunk,
                                   on_admit=lambda rid, slot: self.runner.storage.clear_slot(slot))
        self.sampler = Sampler(self.rt.device, self.rt.dtype)
        self._ids = itertools.count()
        self._rng = random.Random()
        self.n_steps = 0
        self.n_tokens_run = 0
        # the step whose tokens the host has not read yet: (plan, token ids on the device, pinned copy, event)
        self.overlap = bool(overlap) and self.runner.graphs is not None   # replayed graphs are on a CUDA device only
        self._in_flight = None
        self._pinned = []
        self.n_steps_in_vain = 0
        self.n_steps_ahead = 0              # steps launched before the tokens of the step before them were read
        self.n_portion_steps_ahead = 0      # ... of them, steps with prompt portions
        # what the kernels report about themselves is looked at every few steps and when a request has ended
        self.health = KernelHealth(self.rt.dtype) if self.rt.device.type == "cuda" else None
        self.kernel_errors: List[dict] = []
        self._unchecked: List[Request] = []  # ended since the last look that found nothing
        self._checked_up_to = 0              # ... of them, those that ended before the look on its way was asked for
        self._last_look = 0

    # ---- requests -------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None,
                    rid: Optional[Hashable] = None) -> Hashable:
        sampling = sampling or SamplingParams()
        if rid is None:
            rid = next(self._ids)
        seed = sampling.seed if sampling.seed is not None else self._rng.getrandbits(63)
        prompt = [int(t) for t in prompt]
        for t in prompt:
            if not 0 <= t < self.spec.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {self.spec.vocab_size}")
        self.scheduler.add(Request(rid=rid, prompt=prompt, params=sampling, seed=seed))
        return rid

    def abort(self, rid: Hashable):
        return self.scheduler.abort(rid)

    def has_work(self) -> bool:
        return not self.scheduler.idle or self._in_flight is not None

    def warm_up(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """Capture the decode graphs for the given numbers of requests (all, if none is given) before the
        first request comes, so that no request waits for a capture."""
        return self.runner.warm_up(batch_sizes)

    # ---- one scheduler iteration -----------------------------------------------------
    def _launch(self, plan: List[PlannedEntry], before=None):
        """Run the planned step and sample; the token ids stay on the device, a copy is on its way to pinned
        memory.  ``before`` is the launched step whose tokens the host has not read yet: an entry whose token is
        among them takes it from there on the device.  Returns the step as it is kept until its tokens are read."""
        place = {}
        if before is not None and before[1] is not None:
            place = {id(e.request): i for i, e in enumerate(x for x in before[0] if x.samples)}
        entries, sources = [], []
        for e in plan:
            r = e.request
            if e.start + e.n > r.n_tokens:      # the entry reaches past what the host knows: the token on its way
                if e.n != 1 or id(r) not in place:
                    raise RuntimeError(f"request {r.rid!r}: its next token is neither known nor on its way")
                toks, src = [0], place[id(r)]
            else:
                toks, src = r.token_slice(e.start, e.n), -1
            entries.append(StepEntry(r.rid, toks, [e.n - 1] if e.samples else []))
            sources.append(src)
        carried = any(s >= 0 for s in sources)
        logits = self.runner.step(entries, own_output=False, carry=(before[1], sources) if carried else None)
        self.scheduler.advance(plan)
        sampling = [(e, s) for e, s in zip(plan, sources) if e.samples]
        ids = host = event = None
        if sampling:
            pending = [int(s >= 0) for _, s in sampling]
            # a pending token is looked up on the device, where the step before left it
            pending_from = (before[1], [max(s, 0) for _, s in sampling]) if any(pending) else None
            ids = self.sampler.sample(logits, [e.request.params for e, _ in sampling],
                                      [e.request.seed for e, _ in sampling], [e.request for e, _ in sampling],
                                      pending, pending_from=pending_from)
            if self.overlap and ids.device.type == "cuda":
                # the token ids start their way to pinned memory now; an event says when they are there
                host = self._pinned.pop() if self._pinned else \
                    torch.empty((max(self.scheduler.max_batch_size, ids.shape[0]),), dtype=torch.int32).pin_memory()
                host[:ids.shape[0]].copy_(ids, non_blocking=True)
                event = torch.cuda.Event()
                event.record()
        self.n_steps += 1
        self.n_tokens_run += sum(e.n for e in plan)
        return plan, ids, host, event

    def _finish(self, step) -> List[Request]:
        """Read a launched step's tokens and record them; returns the requests that ended with it."""
        plan, ids, host, event = step
        tokens: List[int] = []
        if ids is not None:
            if event is not None:
                event.synchronize()
                tokens = host[:ids.shape[0]].tolist()
                self._pinned.append(host)
            else:
                tokens = ids.cpu().tolist()
        # a request that ended while this step was already on its way ran in vain: it is left out
        alive, kept, it = [], [], iter(tokens)
        for e in plan:
            tok = next(it) if e.samples else None
            if e.request.finish_reason is None:
                alive.append(e)
                if e.samples:
                    kept.append(tok)
            else:
                self.n_steps_in_vain += 1
        return self.scheduler.deliver(alive, kept)

    def _ends_for_sure(self, step) -> bool:
        """Whether a request of the launched step ends with the token that is on its way whatever that token is
        (its last allowed token, or the last position): the step after it is then planned with that known."""
        sch = self.scheduler
        for e in step[0]:
            r = e.request
            if e.samples and r.finish_reason is None and (
                    len(r.output) + r.n_in_flight >= r.params.max_tokens
                    or r.n_tokens + r.n_in_flight >= sch.max_positions):
                return True
        return False

    # ---- what the kernels report about themselves ---------------------------------------
    def _look_at_kernels(self, wait: bool = False) -> List[Request]:
        """Read the kernels' error words if they have arrived (``wait``: ask for them now and wait).  A word that is
        set means that rows of some step since the last clean look were left unwritten: every running request, and
        every request that ended since that look, ends with reason "error"; the words are cleared.  Returns the
        requests that ended here."""
        h = getattr(self, "health", None)
        if h is None:
            return []
        if wait and not h.pending:
            h.queue()
            self._checked_up_to = len(self._unchecked)
        found = h.poll(wait)
        if found is None:
            return []
        if not found:
            del self._unchecked[:self._checked_up_to]
            self._checked_up_to = 0
            return []
        failed = self.flush() if self._in_flight is not None else []
        found.update(h.reset())
        self.kernel_errors.append({"step": self.n_steps, "words": found})
        for r in list(self.scheduler.running):
            self.scheduler.abort(r.rid, reason="error")
            failed.append(r)
        for r in self._unchecked + failed:
            r.finish_reason = "error"
        self._unchecked, self._checked_up_to = [], 0
        return failed

    def _ask_about_kernels(self, ended: Sequence[Request]):
        h = getattr(self, "health", None)
        if h is None:
            return
        self._unchecked.extend(ended)
        if not h.pending and (ended or self.n_steps - self._last_look >= h.every):
            h.queue()
            self._checked_up_to = len(self._unchecked)
            self._last_look = self.n_steps

    def step(self) -> List[Request]:
        """Plan, run and sample one step; returns the requests that are known to have finished.  With
        ``overlap`` the step is launched before the tokens of the one before it are read, where that can be.
        A request may end with reason "error": a kernel reported that it left rows unwritten (``stats()`` says
        which); a request that a call before returned as finished is marked so too if it ended since the last
        look that found nothing."""
        failed = self._look_at_kernels()
        if failed:
            return failed
        finished = self._step()
        self._ask_about_kernels(finished)
        return finished

    def _step(self) -> List[Request]:
        finished: List[Request] = []
        prev, self._in_flight = self._in_flight, None
        if prev is not None and self._ends_for_sure(prev):
            finished += self._finish(prev)
            prev = None
        planned = self.scheduler.plan(may_preempt=prev is None)
        if planned is None:
            # pages are short: the step on its way may end a request; only then is a request's work thrown away
            finished += self._finish(prev)
            prev = None
            planned = self.scheduler.plan()
        plan, ended = planned
        if prev is not None and any(e.start + e.n > e.request.n_tokens for e in plan):
            entries = [StepEntry(e.request.rid, [0] * e.n, []) for e in plan]
            if not self.runner.takes_carried_tokens(entries):
                # this step needs its tokens on the host: read them, and leave out who ended with them
                finished += self._finish(prev)
                prev = None
                plan = [e for e in plan if e.request.finish_reason is None]
        if not plan:
            if prev is not None:
                finished += self._finish(prev)
            return finished + ended
        launched = self._launch(plan, before=prev)
        if prev is not None:
            self.n_steps_ahead += 1
            self.n_portion_steps_ahead += any(e.n > 1 for e in plan)
            finished += self._finish(prev)
        if self.overlap:
            self._in_flight = launched
            return finished + ended
        return finished + ended + self._finish(launched)

    def flush(self) -> List[Request]:
        """Read the tokens of a step that is still on its way; returns the requests that ended with it."""
        prev, self._in_flight = self._in_flight, None
        return self._finish(prev) if prev is not None else []

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 return_requests: bool = False):
        """Generated token ids for every prompt (list of lists, in the order of ``prompts``)."""
        if sampling is None or isinstance(sampling, SamplingParams):
            sampling = [sampling] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        rids = [self.add_request(p, s) for p, s in zip(prompts, sampling)]
        done: Dict[Hashable, Request] = {}
        while len(done) < len(rids) and self.has_work():
            for r in self.step():
                done[r.rid] = r
        for r in self._look_at_kernels(wait=True):      # the device is idle now: this look costs nothing
            done[r.rid] = r
        out = [done[r] for r in rids]
        if return_requests:
            return out
        bad = [r.rid for r in out if r.finish_reason == "error"]
        if bad:
            raise KernelFault(f"requests {bad} ended with an error that a kernel reported: {self.kernel_errors[-1]}")
        return [r.output for r in out]

    def stream(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None):
        """Generated token ids of one prompt, one after the other as the steps bring them (the reference's
        ``run`` prints text as it comes, inferrs/src/run.rs:34-146).  Other requests may be live meanwhile."""
        rid = self.add_request(prompt, sampling)
        request = next(r for r in self.scheduler.waiting if r.rid == rid)
        self.last_streamed = request      # for callers that want the reason of its end afterwards
        sent = 0
        while request.finish_reason is None and self.has_work():
            self.step()
            while sent < len(request.output):
                yield request.output[sent]
                sent += 1
        if request.finish_reason is None:
            self.flush()
        while sent < len(request.output):
            yield request.output[sent]
            sent += 1

    def stats(self) -> dict:
        m = self.runner.manager
        return {
            "steps": self.n_steps,
            "tokens_run": self.n_tokens_run,
            "preemptions": self.scheduler.n_preemptions,
            "steps_in_vain": self.n_steps_in_vain,
            "steps_ahead": self.n_steps_ahead,
            "portion_steps_ahead": self.n_portion_steps_ahead,
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "free_pages": [p.n_free for p in m.pools],
            "pages": [p.n_pages for p in m.pools],
            "cache_bytes": self.runner.storage.total_bytes(),
            "kernel_errors": list(getattr(self, "kernel_errors", [])),
        }
