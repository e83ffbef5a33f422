"""Decode steps as replayed CUDA graphs.

A step in which every request brings one token runs the same kernels with the same shapes every
time; only the numbers in the step's description change.  Such a step is captured once per batch
size (rounded up to a bucket) and replayed: the host then pays for one copy of the description and
one graph launch instead of several hundred kernel launches.  The reference launches every kernel
from the host for every token (inferrs/src/engine.rs:2121-2147).

Captured are exactly the calls that an uncaptured step makes (``Model.forward``), on buffers of
fixed address: the description lives in one fixed int32 buffer, block tables are padded to the
longest context, and the batch is padded with requests that own no pages.

The description of a replayed step is written by the native cache manager straight into pinned host
memory (``ibh_describe_decode``) and reaches the device in one asynchronous copy.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from .batch import StepContext, StepEntry, build_context


def buckets_up_to(n: int) -> List[int]:
    out, b = [], 1
    while b < n:
        out.append(b)
        b *= 2
    out.append(n)
    return out


class _Captured:
    def __init__(self, graph, buffer, logits, launches):
        self.graph, self.buffer, self.logits, self.launches = graph, buffer, logits, launches
        # host side of the description: two pinned copies that take turns as the source of the transfer (a
        # copy may still be waiting in the stream when the next step is described)
        self.staging = [torch.zeros((buffer.numel(),), dtype=torch.int32).pin_memory() for _ in range(2)]
        self.copied = [None, None]          # the event after each pinned copy's last transfer
        self.turn = 0


class DecodeGraphs:
    def __init__(self, runner, max_context: int):
        self.runner = runner
        self.page_size = runner.page_size
        self.fixed_pages = [(max_context + self.page_size - 1) // self.page_size for _ in runner.manager.groups]
        self.max_context = max_context
        self.buckets = buckets_up_to(runner.manager.max_requests)
        self.captured: Dict[int, _Captured] = {}
        self.pool = None

    def bucket_for(self, n: int) -> int:
        return next(b for b in self.buckets if b >= n)

    def _context(self, entries: Sequence[StepEntry], bucket: int, buffer: torch.Tensor) -> StepContext:
        r = self.runner
        ctx = build_context(entries, r.manager, r.storage, r.spec.vocab_size, r.spec.max_positions, r.rt.device,
                            fixed_pages=self.fixed_pages, pad_to=bucket, into=buffer)
        # host numbers that the parts read must not depend on the step: the longest context stands in
        ctx.max_kv_len = self.max_context
        return ctx

    def _buffer_size(self, bucket: int) -> int:
        per_part = (bucket + 4) // 4 * 4
        return 8 * per_part + sum((bucket * p + 3) // 4 * 4 for p in self.fixed_pages) + 16

    # ---- the description of a replayed step -------------------------------------------
    def _describe(self, cap: _Captured, entries: Sequence[StepEntry], bucket: int):
        """Bring the device's description up to date for these entries: native code writes it into pinned
        memory from the cache's book, one asynchronous copy takes it to the device."""
        r = self.runner
        k = cap.turn
        cap.turn ^= 1
        if cap.copied[k] is not None:
            cap.copied[k].synchronize()     # the transfer that last read this pinned copy has been done
        stage = cap.staging[k]
        tokens = [e.tokens[0] for e in entries]
        vocab = r.spec.vocab_size
        code = -1
        if all(isinstance(t, int) and 0 <= t < vocab for t in tokens):
            code, _ = r.manager.describe_decode([e.rid for e in entries], tokens, bucket, self.fixed_pages, vocab,
                                                r.spec.max_positions, stage.data_ptr(), stage.numel())
        if code < 0:
            # something is wrong with an entry: the general builder says what (or builds it, if it can)
            ctx = build_context(entries, r.manager, r.storage, vocab, r.spec.max_positions, torch.device("cpu"),
                                fixed_pages=self.fixed_pages, pad_to=bucket)
            host = ctx.extra["host"]
            stage.numpy()[:host.size] = host
        cap.buffer.copy_(stage, non_blocking=True)
        ev = cap.copied[k] or torch.cuda.Event()
        ev.record()
        cap.copied[k] = ev

    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Logits [wanted rows, vocab] of a step of single tokens; pages are already reserved."""
        bucket = self.bucket_for(len(entries))
        cap = self.captured.get(bucket)
        if cap is None:
            cap = self._capture(entries, bucket)
        else:
            self._describe(cap, entries, bucket)
            cap.graph.replay()
            kernels.count_launches(cap.launches)
        wanted = [i for i, e in enumerate(entries) for _ in e.want]
        if wanted == list(range(len(entries))):
            return cap.logits[:len(entries)]
        if not wanted:
            return cap.logits[:0]
        return cap.logits.index_select(0, torch.tensor(wanted, device=cap.logits.device))

    def _capture(self, entries: Sequence[StepEntry], bucket: int) -> _Captured:
        r = self.runner
        buffer = torch.zeros((self._buffer_size(bucket),), dtype=torch.int32, device=r.rt.device)
        ctx = self._context(entries, bucket, buffer)
        # once outside the capture: libraries initialise, the allocator warms up, and the step's keys are written
        r.model.forward(ctx)
        torch.cuda.synchronize()
        # the captured launches may overlap their neighbours' ends (programmatic dependent launch)
        kernels.set_pdl(True, r.rt.dtype)
        graph = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        # No Python object may be collected while the stream captures: the destructor of an older graph
        # calls into CUDA and would invalidate the capture.
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self.pool):
                logits = r.model.forward(ctx)
        finally:
            kernels.set_pdl(False, r.rt.dtype)
            if was_enabled:
                gc.enable()
        launches = kernels.launch_count() - n0
        if self.pool is None:
            self.pool = graph.pool()
        graph.replay()  # the same step again: it rewrites the same keys and gives the captured output its values
        cap = _Captured(graph, buffer, logits, launches)
        self.captured[bucket] = cap
        return cap
