"""Continuous batching: which requests run in the next step, and with how many tokens.

The reference's loop admits requests while fewer than ``max_batch_size`` are active, runs one
forward pass per sequence per turn, never cuts a prompt (``--max-tokens-per-step`` is parsed and
unused) and fails a request when blocks run out (inferrs/src/engine.rs:1380-1912, :2093-2095).
Here every step is one batch under a token budget:

1. every running request that has one token left to run (a decoded token) gets it, oldest first;
2. running requests in the middle of their prompt get a portion of what is left of the budget;
3. waiting requests are admitted first-come first-served while a state slot, budget and pages for
   their first portion are there.

When pages run out for a token that a running request needs, the *youngest* running request is
preempted: its pages and slot are given back and it returns to the head of the waiting queue with
its prompt and what it has generated so far as its new prompt (it is recomputed later).  A request
that cannot fit even alone is refused when it is added, or ends with reason "length" when it grows
to that size.

The scheduler decides only; it owns no device memory and runs no kernel.  The decisions are made in native
code (``csrc/host_runtime.cpp``, beside the cache's book, which it asks how many pages a plan needs and where it
admits and releases requests); this module is its front: it keeps the requests' tokens, options and results
and follows what the native scheduler decides.
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager, host_library
from ..sampling.params import SamplingParams


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
    handle: int = -1                # the number by which native code knows the request

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
    _ERRORS = {-20: "the prompt is empty", -21: "the prompt leaves no room within the model's positions",
               -22: "the prompt does not fit the cache even alone",
               -23: "a launched step's tokens must be delivered before a plan that may preempt"}
    _REASONS = {1: "stop", 2: "length"}

    def __init__(self, manager: CacheManager, max_batch_size: int, max_tokens_per_step: int,
                 max_positions: int, eos_token_ids: Sequence[int] = (), prefill_chunk: Optional[int] = None,
                 on_admit: Optional[Callable[[Hashable, int], None]] = None):
        """``on_admit(rid, slot)`` is called for every request that a plan admits, a preempted request that
        comes back included, before the plan is returned: whoever owns per-request state of fixed size starts
        it afresh there (a request that is computed again must not find what its first run left)."""
        if max_batch_size <= 0 or max_tokens_per_step <= 0:
            raise SchedulerError("max_batch_size and max_tokens_per_step must be positive")
        self.manager = manager
        self.on_admit = on_admit
        self.max_batch_size = min(max_batch_size, manager.max_requests)
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk or max_tokens_per_step
        self.max_positions = max_positions
        self.eos_token_ids = tuple(int(t) for t in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0
        self._lib = host_library()
        eos = (ctypes.c_int * max(1, len(self.eos_token_ids)))(*self.eos_token_ids)
        self._h = self._lib.ibh_sched_new(manager._h, self.max_batch_size, max_tokens_per_step, self.prefill_chunk,
                                          max_positions, eos, len(self.eos_token_ids))
        if not self._h:
            raise SchedulerError("the native scheduler refused these sizes")
        self._by_handle: Dict[int, Request] = {}
        self._cap = 0
        self._grow(max(64, 2 * self.max_batch_size))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ibh_sched_delete(h)

    def _grow(self, cap: int):
        """Room for the lists that a plan returns."""
        self._cap = cap
        self._rids = (ctypes.c_int64 * cap)()
        self._entries = (ctypes.c_int * (3 * cap))()
        self._lists = [(ctypes.c_int64 * cap)() for _ in range(3)]
        self._counts = [ctypes.c_int() for _ in range(4)]

    @property
    def n_preemptions(self) -> int:
        return self._lib.ibh_sched_n_preemptions(self._h)

    # ---- adding and removing --------------------------------------------------
    def add(self, request: Request):
        p = request.params
        stop = [int(t) for t in p.stop_token_ids]
        request.handle = self.manager.new_handle()
        code = self._lib.ibh_sched_add(self._h, request.handle, len(request.prompt), int(p.max_tokens),
                                       int(bool(p.ignore_eos)), (ctypes.c_int * max(1, len(stop)))(*stop), len(stop))
        if code == -20:
            raise SchedulerError(f"request {request.rid!r}: the prompt is empty")
        if code == -21:
            raise SchedulerError(f"request {request.rid!r}: a prompt of {len(request.prompt)} tokens leaves no room "
                                 f"within the model's {self.max_positions} positions")
        if code == -22:
            raise SchedulerError(f"request {request.rid!r}: a prompt of {len(request.prompt)} tokens does not fit "
                                 f"the cache even alone")
        if code != 0:
            raise SchedulerError(f"request {request.rid!r}: the native scheduler answered {code}")
        request.order = self._arrivals
        self._arrivals += 1
        self._by_handle[request.handle] = request
        self.waiting.append(request)
        if len(self._by_handle) + 8 > self._cap:
            self._grow(2 * self._cap)

    def abort(self, rid: Hashable, reason: str = "cancelled") -> Optional[Request]:
        """Take the request out (its pages and slot are free again); it ends with ``reason``."""
        for r in list(self.running) + list(self.waiting):
            if r.rid == rid:
                was = self._lib.ibh_sched_abort(self._h, r.handle)
                if was == 1:
                    self.running.remove(r)
                    self.manager.forget(rid)
                elif was == 2:
                    self.waiting.remove(r)
                else:
                    raise SchedulerError(f"request {rid!r}: the native scheduler does not know it")
                del self._by_handle[r.handle]
                r.finish_reason = reason
                return r
        return None

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- planning ---------------------------------------------------------------
    def plan(self, may_preempt: bool = True) -> Optional[Tuple[List[PlannedEntry], List[Request]]]:
        """(entries of the next step, requests that ended while planning because they outgrew the cache).

        Pages are not taken here; the step function reserves exactly what this plan was checked for.
        ``may_preempt=False``: None, with nothing changed, if the step cannot be planned without taking a running
        request's pages away or ending one (a caller that has a step on its way asks so, reads that step's tokens
        and plans again).
        """
        c = self._counts
        code = self._lib.ibh_sched_plan(self._h, int(bool(may_preempt)), self._cap, self._rids, self._entries,
                                        ctypes.byref(c[0]), self._lists[0], ctypes.byref(c[1]), self._lists[1],
                                        ctypes.byref(c[2]), self._lists[2], ctypes.byref(c[3]))
        if code == 1:
            return None
        if code in self._ERRORS:
            raise SchedulerError(self._ERRORS[code])
        if code != 0:
            raise SchedulerError(f"plan: the native scheduler answered {code}")
        # follow what happened, in the order in which it can have happened: preemptions and ends come before
        # the admissions of the plan that was made in the end
        for h in self._lists[0][:c[1].value]:
            v = self._by_handle[h]
            self.running.remove(v)
            self.manager.forget(v.rid)
            v.n_computed = 0
            v.n_preempted += 1
            self.waiting.appendleft(v)
        ended: List[Request] = []
        for h in self._lists[1][:c[2].value]:
            r = self._by_handle.pop(h)
            self.running.remove(r)
            self.manager.forget(r.rid)
            r.finish_reason = "length"
            ended.append(r)
        for h in self._lists[2][:c[3].value]:
            r = self.waiting.popleft()
            if r.handle != h:
                raise SchedulerError("the front and the native scheduler disagree about the waiting queue")
            self.manager.adopt(r.rid, h)
            self.running.append(r)
            if self.on_admit is not None:
                self.on_admit(r.rid, self.manager.slot(r.rid))
        e = self._entries
        plan = [PlannedEntry(self._by_handle[self._rids[i]], e[3 * i], e[3 * i + 1], bool(e[3 * i + 2]))
                for i in range(c[0].value)]
        return plan, ended

    # ---- after the step ---------------------------------------------------------
    def advance(self, plan: Sequence[PlannedEntry]):
        """The planned step has been launched: its tokens count as run, and every entry that samples has a token on
        its way that the host does not know yet."""
        n = len(plan)
        if n == 0:
            return
        code = self._lib.ibh_sched_advance(self._h, n, (ctypes.c_int64 * n)(*[e.request.handle for e in plan]),
                                           (ctypes.c_int * n)(*[e.n for e in plan]),
                                           (ctypes.c_int * n)(*[int(e.samples) for e in plan]))
        if code != 0:
            raise SchedulerError(f"advance: the native scheduler answered {code}")
        for e in plan:
            e.request.n_computed += e.n
            if e.samples:
                e.request.n_in_flight += 1

    def deliver(self, plan: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[Request]:
        """The tokens of a launched step have arrived: ``sampled`` holds one per planned entry with ``samples``,
        in plan order.  Returns the requests that finished; their pages and slots are free again."""
        sampling = [e.request for e in plan if e.samples]
        n = len(sampling)
        if n == 0:
            return []
        tokens = [int(t) for t in sampled]
        if len(tokens) != n:
            raise SchedulerError(f"deliver: {len(tokens)} tokens for {n} entries that sample")
        reasons = (ctypes.c_int * n)()
        code = self._lib.ibh_sched_deliver(self._h, n, (ctypes.c_int64 * n)(*[r.handle for r in sampling]),
                                           (ctypes.c_int * n)(*tokens), reasons)
        if code != 0:
            raise SchedulerError(f"deliver: the native scheduler answered {code}")
        finished: List[Request] = []
        for r, tok, reason in zip(sampling, tokens, reasons):
            r.n_in_flight -= 1
            r.output.append(tok)
            if reason:
                r.finish_reason = self._REASONS[reason]
                self.running.remove(r)
                self.manager.forget(r.rid)
                del self._by_handle[r.handle]
                finished.append(r)
        return finished

    def update(self, plan: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[Request]:
        """Record a step whose tokens are known: :meth:`advance` and :meth:`deliver` in one."""
        self.advance(plan)
        return self.deliver(plan, sampled)

    def check(self):
        """The front's view of every request against the native scheduler's (for tests)."""
        out = (ctypes.c_int * 6)()
        for state, group in ((0, self.waiting), (1, self.running)):
            for r in group:
                if self._lib.ibh_sched_counts(self._h, r.handle, out) != 0:
                    raise SchedulerError(f"request {r.rid!r} is unknown to the native scheduler")
                mine = (len(r.prompt), len(r.output), r.n_computed, r.n_in_flight, r.n_preempted, state)
                if tuple(out) != mine:
                    raise SchedulerError(f"request {r.rid!r}: front {mine}, native {tuple(out)}")
        if (self._lib.ibh_sched_n_waiting(self._h), self._lib.ibh_sched_n_running(self._h)) != \
                (len(self.waiting), len(self.running)):
            raise SchedulerError("the front and the native scheduler count their requests differently")
