"""A plain model of the scheduler: the decisions that the native scheduler makes, written down in Python.

The tests drive this model (over the plain cache book, ``plain_cache.py``) and the product's scheduler (native
code over the native cache book) with the same requests and tokens; every plan, every preemption, every end
and the order of page reuse must agree.

Every step is one batch under a token budget:

1. every running request that has one token left to run (a decoded token) gets it, oldest first;
2. running requests in the middle of their prompt get a portion of what is left of the budget;
3. waiting requests are admitted first-come first-served while a state slot, budget and pages for
   their first portion are there.

When pages run out for a token that a running request needs, the youngest running request is preempted: its
pages and slot are given back and it returns to the head of the waiting queue; all its tokens are run again
later.  A request that cannot fit even alone is refused when it is added, or ends with reason "length" when it
grows to that size.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from inferrs_b200.sampling.params import SamplingParams


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    seed: int
    output: List[int] = field(default_factory=list)
    n_computed: int = 0             # tokens whose keys and values are in the cache (or will be after a launched step)
    n_in_flight: int = 0            # tokens that launched steps have sampled and the host has not read yet
    finish_reason: Optional[str] = None
    n_preempted: int = 0
    order: int = 0                  # arrival number: smaller is older

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def n_pending(self) -> int:
        """Tokens that still have to run; one of them may be a token that is on its way from the device."""
        return len(self.prompt) + len(self.output) + self.n_in_flight - self.n_computed

    def token_slice(self, start: int, n: int) -> List[int]:
        """tokens[start:start + n] without building the whole list."""
        p = len(self.prompt)
        if start >= p:
            return self.output[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - p]

    def tail(self, n: int) -> List[int]:
        """The last n tokens (prompt and generated)."""
        if n <= 0:
            return []
        if n <= len(self.output):
            return self.output[-n:]
        return self.prompt[-(n - len(self.output)):] + self.output


@dataclass
class PlannedEntry:
    request: Request
    start: int        # index of the first token of the portion within request.tokens
    n: int            # number of tokens
    samples: bool     # the portion reaches the request's last token: its last row is sampled


class SchedulerError(ValueError):
    pass


class Scheduler:
    def __init__(self, manager, max_batch_size: int, max_tokens_per_step: int,
                 max_positions: int, eos_token_ids: Sequence[int] = (), prefill_chunk: Optional[int] = None):
        if max_batch_size <= 0 or max_tokens_per_step <= 0:
            raise SchedulerError("max_batch_size and max_tokens_per_step must be positive")
        self.manager = manager
        self.max_batch_size = min(max_batch_size, manager.max_requests)
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk or max_tokens_per_step
        self.max_positions = max_positions
        self.eos_token_ids = tuple(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0
        self.n_preemptions = 0

    # ---- adding and removing --------------------------------------------------
    def _pages_alone(self, n_tokens: int) -> bool:
        pages = (n_tokens + self.manager.page_size - 1) // self.manager.page_size
        return all(pages <= pool.n_pages for pool in self.manager.pools)

    def add(self, request: Request):
        if not request.prompt:
            raise SchedulerError(f"request {request.rid!r}: the prompt is empty")
        if len(request.prompt) >= self.max_positions:
            raise SchedulerError(f"request {request.rid!r}: a prompt of {len(request.prompt)} tokens leaves no room "
                                 f"within the model's {self.max_positions} positions")
        if not self._pages_alone(len(request.prompt) + 1):
            raise SchedulerError(f"request {request.rid!r}: a prompt of {len(request.prompt)} tokens does not fit "
                                 f"the cache even alone")
        request.order = self._arrivals
        self._arrivals += 1
        self.waiting.append(request)

    def abort(self, rid: Hashable) -> Optional[Request]:
        for r in list(self.running):
            if r.rid == rid:
                self.running.remove(r)
                self.manager.release(rid)
                r.finish_reason = "cancelled"
                return r
        for r in list(self.waiting):
            if r.rid == rid:
                self.waiting.remove(r)
                r.finish_reason = "cancelled"
                return r
        return None

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- planning ---------------------------------------------------------------
    def _preempt_youngest(self, keep: Request) -> bool:
        victims = [r for r in self.running if r is not keep]
        if not victims:
            return False
        v = max(victims, key=lambda r: r.order)
        self.running.remove(v)
        self.manager.release(v.rid)
        v.n_computed = 0
        v.n_preempted += 1
        self.n_preemptions += 1
        self.waiting.appendleft(v)
        return True

    def plan(self, may_preempt: bool = True) -> Optional[Tuple[List[PlannedEntry], List[Request]]]:
        """(entries of the next step, requests that ended while planning because they outgrew the cache).

        Pages are not taken here; the step function reserves exactly what this plan was checked for.
        ``may_preempt=False``: None, with nothing changed, if the step cannot be planned without taking a running
        request's pages away or ending one (a caller that has a step on its way asks so, reads that step's tokens
        and plans again).
        """
        ended: List[Request] = []
        while True:
            budget = self.max_tokens_per_step
            free = [pool.n_free for pool in self.manager.pools]   # pages left once the plan so far is served
            plan: List[PlannedEntry] = []
            starved: Optional[Request] = None

            def fits(rid, n) -> bool:
                need = self.manager.pages_needed(rid, n)
                if any(need[g] > free[g] for g in range(len(free))):
                    return False
                for g in range(len(free)):
                    free[g] -= need[g]
                return True

            by_age = sorted(self.running, key=lambda r: r.order)
            # decoded tokens first, then portions of prompts, oldest first
            order = [r for r in by_age if r.n_pending == 1] + [r for r in by_age if r.n_pending > 1]
            counts = []
            for r in order:
                if budget <= 0:
                    break
                n = min(r.n_pending, budget, self.prefill_chunk)
                counts.append(n)
                budget -= n
            order = order[:len(counts)]
            fitted = self.manager.fit_in_order([r.rid for r in order], counts, free) if order else 0
            for r, n in zip(order[:fitted], counts[:fitted]):
                plan.append(PlannedEntry(r, r.n_computed, n, n == r.n_pending))
            if fitted < len(order):
                starved = order[fitted]
                budget += sum(counts[fitted:])
            if starved is not None:
                if not may_preempt:
                    return None
                if any(r.n_in_flight for r in self.running):
                    raise SchedulerError("a launched step's tokens must be delivered before a plan that may preempt")
                if self._preempt_youngest(keep=starved):
                    continue  # plan again with the pages that came back
                # the request is alone and still does not fit: it has outgrown the cache
                self.running.remove(starved)
                self.manager.release(starved.rid)
                starved.finish_reason = "length"
                ended.append(starved)
                continue
            # admission, first come first served
            while self.waiting and budget > 0 and len(self.running) < self.max_batch_size \
                    and self.manager.n_free_slots > 0:
                r = self.waiting[0]
                n = min(r.n_pending, budget, self.prefill_chunk)
                self.manager.admit(r.rid)
                if not fits(r.rid, n):
                    self.manager.release(r.rid)
                    break
                self.waiting.popleft()
                self.running.append(r)
                plan.append(PlannedEntry(r, r.n_computed, n, n == r.n_pending))
                budget -= n
            return plan, ended

    # ---- after the step ---------------------------------------------------------
    def stop_reason(self, r: Request, token: int) -> Optional[str]:
        if not r.params.ignore_eos and (token in self.eos_token_ids or token in r.params.stop_token_ids):
            return "stop"
        if len(r.output) >= r.params.max_tokens:
            return "length"
        if len(r.prompt) + len(r.output) >= self.max_positions:
            return "length"
        return None

    def advance(self, plan: Sequence[PlannedEntry]):
        """The planned step has been launched: its tokens count as run, and every entry that samples has a token on
        its way that the host does not know yet."""
        for e in plan:
            e.request.n_computed += e.n
            if e.samples:
                e.request.n_in_flight += 1

    def deliver(self, plan: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[Request]:
        """The tokens of a launched step have arrived: ``sampled`` holds one per planned entry with ``samples``,
        in plan order.  Returns the requests that finished; their pages and slots are free again."""
        finished: List[Request] = []
        it = iter(sampled)
        for e in plan:
            if not e.samples:
                continue
            r = e.request
            tok = int(next(it))
            r.n_in_flight -= 1
            r.output.append(tok)
            reason = self.stop_reason(r, tok)
            if reason is not None:
                r.finish_reason = reason
                self.running.remove(r)
                self.manager.release(r.rid)
                finished.append(r)
        return finished

    def update(self, plan: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[Request]:
        """Record a step whose tokens are known: :meth:`advance` and :meth:`deliver` in one."""
        self.advance(plan)
        return self.deliver(plan, sampled)
