"""Steps as replayed CUDA graphs: decode steps (``DecodeGraphs``) and steps with prompt portions (``PortionGraphs``).

A step in which every request brings one token runs the same kernels with the same shapes every
time; only the numbers in the step's description change.  Such a step is captured once per batch
size (rounded up to a bucket) and replayed: the host then pays for one copy of the description and
one graph launch instead of several hundred kernel launches.  The reference launches every kernel
from the host for every token (inferrs/src/engine.rs:2121-2147).

Captured are exactly the calls that an uncaptured step makes (``Model.forward``), on buffers of
fixed address: the description lives in one fixed int32 buffer, block tables are padded to the
longest context, and the batch is padded with requests that own no pages.

The description of a replayed step is written by the native cache manager straight into pinned host
memory (``ibh_describe_decode``, ``ibh_describe_step``) and reaches the device in one asynchronous copy.  A
token that an earlier step sampled and the host has not read yet is named there by its place in that step's
output; a small kernel puts the id itself there before the graph is replayed (``name_carried_tokens``).
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


def name_carried_tokens(stage: torch.Tensor, entries: Sequence[StepEntry], sources: Sequence[int]):
    """In a description in pinned memory, replace the token id of every entry that has a source (>= 0) by the
    stand-in -1 - source: ``kernels.resolve_tokens`` puts the token itself there on the device.  Such an entry
    brings exactly one token; the token ids lead the description, in the order of the entries."""
    view = stage.numpy()
    row = 0
    for e, src in zip(entries, sources):
        if src >= 0:
            if len(e.tokens) != 1:
                raise ValueError(f"request {e.rid!r}: only a single token can be taken from the step before")
            view[row] = -1 - src
        row += len(e.tokens)
    return row


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
    def _describe(self, cap: _Captured, entries: Sequence[StepEntry], bucket: int, carry=None):
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
        if carry is not None:
            name_carried_tokens(stage, entries, carry[1])
        cap.buffer.copy_(stage, non_blocking=True)
        ev = cap.copied[k] or torch.cuda.Event()
        ev.record()
        cap.copied[k] = ev
        if carry is not None:
            kernels.resolve_tokens(cap.buffer[:len(entries)], carry[0], r.rt.dtype)

    def run(self, entries: Sequence[StepEntry], carry=None) -> torch.Tensor:
        """Logits [wanted rows, vocab] of a step of single tokens; pages are already reserved.  ``carry`` is
        (int32 token ids on the device, for every entry its place among them or -1): an entry with a place
        takes its token from there, in stream order, and its own token id is a stand-in; so the step can be
        launched before the host has seen the tokens that the step before it sampled."""
        bucket = self.bucket_for(len(entries))
        cap = self.captured.get(bucket)
        if cap is None:
            cap = self._capture(entries, bucket, run=carry is None)
            if carry is None:
                return self._wanted(cap, entries)
        self._describe(cap, entries, bucket, carry)
        cap.graph.replay()
        kernels.count_launches(cap.launches)
        return self._wanted(cap, entries)

    @staticmethod
    def _wanted(cap: _Captured, entries: Sequence[StepEntry]) -> torch.Tensor:
        wanted = [i for i, e in enumerate(entries) for _ in e.want]
        if wanted == list(range(len(entries))):
            return cap.logits[:len(entries)]
        if not wanted:
            return cap.logits[:0]
        return cap.logits.index_select(0, torch.tensor(wanted, device=cap.logits.device))

    def _capture(self, entries: Sequence[StepEntry], bucket: int, run: bool = True) -> _Captured:
        """Capture the step of these entries.  ``run``: also run it for good (one replay); a caller that still has to
        complete the description on the device replays it itself, and a step must run for good exactly once (a
        mixer's fixed-size state moves with every run)."""
        r = self.runner
        buffer = torch.zeros((self._buffer_size(bucket),), dtype=torch.int32, device=r.rt.device)
        ctx = self._context(entries, bucket, buffer)
        # once outside the capture: libraries initialise, the allocator warms up, and the step's keys are written.
        # Writing the same keys twice changes nothing, but a mixer's fixed-size state would move twice: it is put
        # back before the step runs for good (the replay below).
        saved = r.storage.snapshot_states()
        r.model.forward(ctx)
        r.storage.restore_states(saved)
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
        if run:
            graph.replay()  # the step for good: it rewrites the same keys and gives the captured output its values
        cap = _Captured(graph, buffer, logits, launches)
        self.captured[bucket] = cap
        return cap


class PortionGraphs:
    """Steps with prompt portions (alone or beside decoded tokens) as replayed graphs too.

    Such a step is padded to a fixed shape: its rows to the next of a few row counts (the added rows belong to
    one padding request without pages: they write nothing to the cache and nobody reads what they compute), its
    requests to the most the cache admits plus that one, its wanted places to as many.  The attention kernels
    get their tiles from a list of fixed length in the description, in which -1 marks a place without a tile.  A place
    without a tile still costs the launch of a CTA, and a list with room for every request that the cache admits
    would have hundreds of them; so there is a captured step for each of a few numbers of requests that may bring
    tiles (``TILE_PADS``), and a step is replayed by the smallest one that holds it.
    What the host pays per step is then the description and one graph launch instead of a dozen launches per
    layer; for small models and short portions that is the difference between a step bound by the host and one
    bound by the GPU.  The first step of every row count runs once plainly (which also tells which tile sizes
    the model's attention layers ask for) and is then captured.
    """

    ROW_BUCKETS = (32, 64, 128, 256, 512, 1024, 2048, 4096)
    TILE_PADS = (8,)                 # ... and as many requests as the cache admits

    def __init__(self, runner, decode: DecodeGraphs, max_rows: int):
        self.runner = runner
        self.decode = decode                      # shares its memory pool and its limits
        self.fixed_pages = decode.fixed_pages
        self.max_context = decode.max_context
        self.n_requests = runner.manager.max_requests + 1
        self.n_wanted = max(self.n_requests, 64)   # wanted places that a captured step provides
        self.buckets = [b for b in self.ROW_BUCKETS if b <= max(max_rows, self.ROW_BUCKETS[0])]
        self.tile_pads = [t for t in self.TILE_PADS if t < self.n_requests] + [self.n_requests]
        self.captured: Dict[int, Dict[int, _Captured]] = {}      # row count -> requests that may bring tiles -> step
        # per row count: the (tokens per tile, portions only) pairs that the attention layers ask for at that size
        self.tile_sizes: Dict[int, list] = {}

    def bucket_for(self, n_rows: int) -> Optional[int]:
        return next((b for b in self.buckets if b >= n_rows), None)

    def takes(self, entries: Sequence[StepEntry]) -> bool:
        n_rows = sum(len(e.tokens) for e in entries)
        n_wanted = sum(len(e.want) for e in entries)
        m = self.runner.manager
        return (self.bucket_for(n_rows) is not None and len(entries) < self.n_requests and n_wanted <= self.n_wanted
                and all(m.n_tokens(e.rid) + len(e.tokens) <= self.max_context for e in entries))

    def tile_pad_for(self, entries: Sequence[StepEntry], bucket: int) -> int:
        """The smallest provided number of requests with tiles that holds this step's: the requests that bring more
        than one token, or all of them if some attention layer cuts single tokens into tiles too."""
        sizes = self.tile_sizes.get(bucket)
        if sizes is not None and all(portions_only for _, portions_only in sizes):
            n = sum(len(e.tokens) > 1 for e in entries)
        else:
            n = len(entries)
        return next(t for t in self.tile_pads if t >= n)

    def _build(self, entries, bucket, tile_pad, device, into=None) -> StepContext:
        r = self.runner
        ctx = build_context(entries, r.manager, r.storage, r.spec.vocab_size, r.spec.max_positions, device,
                            fixed_pages=self.fixed_pages, into=into, pad_rows=bucket, pad_requests=self.n_requests,
                            pad_wanted=self.n_wanted, tile_sizes=self.tile_sizes[bucket], tile_pad=tile_pad)
        ctx.max_kv_len = self.max_context
        return ctx

    def run(self, entries: Sequence[StepEntry], carry=None) -> torch.Tensor:
        """Logits [wanted rows, vocab]; pages are already reserved.  ``carry`` as in :meth:`DecodeGraphs.run`."""
        r = self.runner
        n_rows = sum(len(e.tokens) for e in entries)
        bucket = self.bucket_for(n_rows)
        n_wanted = sum(len(e.want) for e in entries)
        self._learn_tile_sizes(entries, bucket)
        tile_pad = self.tile_pad_for(entries, bucket)
        cap = self.captured.get(bucket, {}).get(tile_pad)
        if cap is None:
            cap = self._capture(entries, bucket, tile_pad, run=carry is None)
            if carry is None:
                return cap.logits[:n_wanted]
        k = cap.turn
        cap.turn ^= 1
        if cap.copied[k] is not None:
            cap.copied[k].synchronize()
        stage = cap.staging[k]
        try:
            code, _ = r.manager.describe_step(
                [e.rid for e in entries], [e.tokens for e in entries], [e.want for e in entries], bucket,
                self.n_requests, self.n_wanted, self.fixed_pages, self.tile_sizes[bucket], tile_pad, r.spec.vocab_size,
                r.spec.max_positions, stage.data_ptr(), stage.numel())
        except (TypeError, ValueError, OverflowError):
            code = -1
        if code < 0:
            # something is wrong with an entry: the general builder says what (or builds it, if it can)
            host = self._build(entries, bucket, tile_pad, torch.device("cpu")).extra["host"]
            stage.numpy()[:host.size] = host
        if carry is not None:
            name_carried_tokens(stage, entries, carry[1])
        cap.buffer.copy_(stage, non_blocking=True)
        ev = cap.copied[k] or torch.cuda.Event()
        ev.record()
        cap.copied[k] = ev
        if carry is not None:
            kernels.resolve_tokens(cap.buffer[:n_rows], carry[0], r.rt.dtype)
        cap.graph.replay()
        kernels.count_launches(cap.launches)
        return cap.logits[:n_wanted]

    def _learn_tile_sizes(self, entries: Sequence[StepEntry], bucket: int):
        r = self.runner
        if bucket not in self.tile_sizes:
            # once plainly: the attention layers ask the context for their tiles, which tells their sizes (they may
            # depend on how many rows the step has: the plain step says that it stands for the padded one)
            plain = build_context(entries, r.manager, r.storage, r.spec.vocab_size, r.spec.max_positions, r.rt.device)
            plain.extra["dispatch_rows"] = bucket
            saved = r.storage.snapshot_states()     # see DecodeGraphs._capture
            r.model.forward(plain)
            r.storage.restore_states(saved)
            self.tile_sizes[bucket] = sorted(k[1:] for k in plain.extra
                                             if isinstance(k, tuple) and k[0] == "attention_tiles")

    def _capture(self, entries: Sequence[StepEntry], bucket: int, tile_pad: int, run: bool = True) -> _Captured:
        r = self.runner                     # ``run`` as in DecodeGraphs._capture
        size = self._build(entries, bucket, tile_pad, torch.device("cpu")).extra["host"].size
        buffer = torch.zeros((size + 16,), dtype=torch.int32, device=r.rt.device)
        ctx = self._build(entries, bucket, tile_pad, r.rt.device, into=buffer)
        saved = r.storage.snapshot_states()
        r.model.forward(ctx)
        r.storage.restore_states(saved)
        torch.cuda.synchronize()
        kernels.set_pdl(True, r.rt.dtype)
        graph = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        gc.collect()                # see DecodeGraphs._capture
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self.decode.pool):
                logits = r.model.forward(ctx)
        finally:
            kernels.set_pdl(False, r.rt.dtype)
            if was_enabled:
                gc.enable()
        launches = kernels.launch_count() - n0
        if self.decode.pool is None:
            self.decode.pool = graph.pool()
        if run:
            graph.replay()
        cap = _Captured(graph, buffer, logits, launches)
        self.captured.setdefault(bucket, {})[tile_pad] = cap
        return cap
