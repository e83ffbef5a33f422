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

from ..runtime import Runtime, parse_dtype
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .loading import load_model_dir, random_model
from .runner import ModelRunner
from .scheduler import PlannedEntry, Request, Scheduler


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
    overlap              decode steps are launched one ahead: while the device runs a step, the host reads the
                         tokens of the step before and plans; a request that turns out to have ended runs one
                         step in vain.  Results are the same; ``step`` then reports a request's end one call later.
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
        self.max_seq_len = min(max_seq_len, spec.max_positions) if max_seq_len else spec.max_positions
        if num_blocks is None:
            num_blocks = self._blocks_for_fraction(spec, block_size, paged_attention, max_batch_size)
        self.runner = ModelRunner(spec, weights, self.rt, page_size=block_size, n_pages=num_blocks,
                                  max_requests=max_batch_size, max_context=self.max_seq_len)
        self.scheduler = Scheduler(self.runner.manager, max_batch_size, max_tokens_per_step, self.max_seq_len,
                                   spec.eos_token_ids, prefill_chunk)
        self.sampler = Sampler(self.rt.device, self.rt.dtype)
        self._ids = itertools.count()
        self._rng = random.Random()
        self.n_steps = 0
        self.n_tokens_run = 0
        # the step whose tokens the host has not read yet: (plan, token ids on the device, pinned copy, event)
        self.overlap = bool(overlap) and self.rt.device.type == "cuda" and self.runner.graphs is not None
        self._in_flight = None
        self._pinned = []
        self.n_steps_in_vain = 0

    def _blocks_for_fraction(self, spec, block_size, fraction, max_batch_size) -> int:
        from .model import cache_needs
        if not 0.0 < fraction <= 1.0:
            raise ValueError(f"paged_attention must be in (0, 1], got {fraction}")
        kv_needs, _ = cache_needs(spec)
        elem = torch.empty((), dtype=self.rt.dtype).element_size()
        per_page = sum(2 * n.n_kv_heads * n.head_dim * block_size * elem for n in kv_needs.values())
        if self.rt.device.type != "cuda":
            raise RuntimeError("num_blocks must be given when the cache is not on a CUDA device")
        free, _total = torch.cuda.mem_get_info(self.rt.device)
        blocks = int(free * fraction) // max(per_page, 1)
        # no request can use more than max_positions tokens: more pages than that per slot are never touched
        useful = max_batch_size * ((self.max_seq_len + block_size - 1) // block_size)
        blocks = min(blocks, useful)
        if blocks < 1:
            raise RuntimeError("no memory is left for the cache")
        return blocks

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
    def _launch(self, plan: List[PlannedEntry], device_tokens: Optional[torch.Tensor] = None, pending: int = 0):
        """Run the planned step and sample; the token ids stay on the device, a copy is on its way to pinned
        memory.  Returns the step as it is kept until its tokens are read."""
        entries = []
        for e in plan:
            toks = [0] if device_tokens is not None else e.request.token_slice(e.start, e.n)
            entries.append(StepEntry(e.request.rid, toks, [e.n - 1] if e.samples else []))
        logits = self.runner.step(entries, own_output=False, device_tokens=device_tokens)
        sampling = [e for e in plan if e.samples]
        ids = host = event = None
        if sampling:
            ids = self.sampler.sample(logits, [e.request.params for e in sampling],
                                      [e.request.seed for e in sampling], [e.request for e in sampling], pending,
                                      device_tokens)
            if self.overlap:
                host = self._pinned.pop() if self._pinned else \
                    torch.empty((self.scheduler.max_batch_size,), dtype=torch.int32).pin_memory()
                host[:ids.shape[0]].copy_(ids, non_blocking=True)
                event = torch.cuda.Event()
                event.record()
        self.n_steps += 1
        self.n_tokens_run += sum(e.n for e in plan)
        return plan, ids, host, event

    def _finish(self, step) -> List[Request]:
        """Read a launched step's tokens and record it; returns the requests that ended with it."""
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
        return self.scheduler.update(alive, kept)

    def _next_decode_plan(self, step) -> Optional[List[PlannedEntry]]:
        """The step after ``step`` if it can be told before ``step``'s tokens are known: every running request has
        just been sampled and brings exactly the sampled token next.  None if anything else may happen (a prompt
        that can be let in or is under way, too few pages): then the tokens are read first."""
        plan, ids, _, _ = step
        sch = self.scheduler
        if ids is None or len(plan) != len(sch.running) or not all(e.samples for e in plan):
            return None
        # a waiting request that could be let in now needs a planned step; one that finds no room anyway (all
        # slots taken) waits a step longer for the slot of a request that is just ending
        if sch.waiting and len(sch.running) < sch.max_batch_size and self.runner.manager.n_free_slots > 0:
            return None
        nxt = []
        for e in plan:
            r = e.request
            if r.finish_reason is not None:
                return None
            # with the token that is on its way the request has len(output) + 1 tokens: does it go on after it?
            if len(r.output) + 1 >= r.params.max_tokens or r.n_tokens + 1 >= sch.max_positions:
                return None
            nxt.append(PlannedEntry(r, r.n_tokens, 1, True))
        free = [pool.n_free for pool in self.runner.manager.pools]
        # the cache has this step's token committed already: one more token each
        if self.runner.manager.fit_in_order([e.request.rid for e in nxt], [1] * len(nxt), free) != len(nxt):
            return None
        if not self.runner.takes_device_tokens([StepEntry(e.request.rid, [0], [0]) for e in nxt]):
            return None
        return nxt

    def step(self) -> List[Request]:
        """Plan, run and sample one step; returns the requests that are known to have finished.  With
        ``overlap`` the step is launched before the tokens of the one before it are read, where that can be."""
        finished: List[Request] = []
        prev, self._in_flight = self._in_flight, None
        if prev is not None:
            nxt = self._next_decode_plan(prev)
            if nxt is not None:
                self._in_flight = self._launch(nxt, device_tokens=prev[1], pending=1)
                return self._finish(prev)
            finished = self._finish(prev)
        plan, ended = self.scheduler.plan()
        if not plan:
            return finished + ended
        launched = self._launch(plan)
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
        out = [done[r] for r in rids]
        return out if return_requests else [r.output for r in out]

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
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "free_pages": [p.n_free for p in m.pools],
            "pages": [p.n_pages for p in m.pools],
            "cache_bytes": self.runner.storage.total_bytes(),
        }
