"""The step function: run the tokens it is given, as one batch, from the cache.

``ModelRunner`` owns the model, the cache's device memory and its book-keeping.
``step`` takes a list of (request, its next tokens, wanted places), reserves the
pages, runs only those tokens through every scheduled layer, and returns the
logits at the wanted places.  Portions of prompts and single decoded tokens may
stand side by side; a prompt may be cut anywhere.

The reference's nearest counterparts are ``CausalLM::forward_paged``
(inferrs-models/src/models/mod.rs:169-339) driven per sequence by
``cb_prefill`` / ``cb_decode_step`` (inferrs/src/engine.rs:2074-2147).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..cache.storage import CacheStorage
from ..parts.spec import ModelSpec
from ..runtime import Runtime
from .batch import StepContext, StepEntry, build_context
from .model import Model, cache_needs


class ModelRunner:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime, page_size: int,
                 n_pages: Optional[int], max_requests: int, use_graphs: Optional[bool] = None,
                 max_context: Optional[int] = None, graph_rows: int = 2048, cache_fraction: float = 0.9,
                 consume_weights: bool = False):
        """``n_pages`` None: the cache gets ``cache_fraction`` of the device memory that is free once the model
        stands (but no more pages than ``max_requests`` requests of ``max_context`` tokens can use).
        ``consume_weights``: the ``weights`` dictionary is emptied once the model is built; the parts keep what
        they use, and the tensors that were fused into others (q/k/v, gate/up) are given back before the cache is
        sized."""
        self.spec = spec
        self.rt = rt
        self.model = Model(spec, weights, rt, consume=consume_weights)
        kv_needs, state_needs = cache_needs(spec)
        if consume_weights:
            weights.clear()
        if n_pages is None:
            n_pages = self._pages_for_fraction(kv_needs, page_size, cache_fraction, max_requests,
                                               min(max_context or spec.max_positions, spec.max_positions))
        self.storage = CacheStorage(kv_needs, state_needs, page_size, n_pages, max_requests, rt.dtype, rt.device)
        self.manager = CacheManager(self.storage.layouts, page_size, self.storage.n_pages, max_requests)
        self.page_size = page_size
        self.steps_run = 0
        # decode steps are replayed as CUDA graphs when every part says its launches do not depend on
        # host-side values of the step (``graph_safe``)
        parts = [p for b in self.model.blocks for p in b.parts()] + [self.model.final_norm]
        safe = all(getattr(p, "graph_safe", False) for p in parts)
        if use_graphs is None:
            use_graphs = rt.device.type == "cuda"
        self.graphs = None
        self.portion_graphs = None     # steps with prompt portions of up to ``graph_rows`` rows (0: never)
        if use_graphs and safe and rt.device.type == "cuda":
            from .graphs import DecodeGraphs, PortionGraphs
            limit = min(max_context or spec.max_positions, spec.max_positions, n_pages * page_size)
            self.graphs = DecodeGraphs(self, limit)
            if graph_rows > 0:
                self.portion_graphs = PortionGraphs(self, self.graphs, graph_rows)

    def _pages_for_fraction(self, kv_needs, page_size: int, fraction: float, max_requests: int, max_context: int) -> int:
        """Pages that ``fraction`` of the memory that is free right now pays for (the reference sizes its cache as a
        fraction of memory too, inferrs-models/src/kv_cache.rs:44-65, inferrs/src/engine.rs:944-1000)."""
        if not 0.0 < fraction <= 1.0:
            raise ValueError(f"the cache's fraction of free memory must be in (0, 1], got {fraction}")
        if self.rt.device.type != "cuda":
            raise RuntimeError("the number of pages must be given when the cache is not on a CUDA device")
        import gc
        gc.collect()
        torch.cuda.empty_cache()        # what the loader and the fusing of tensors have given back
        elem = torch.empty((), dtype=self.rt.dtype).element_size()
        per_page = sum(2 * n.n_kv_heads * n.head_dim * page_size * elem for n in kv_needs.values())
        free, _total = torch.cuda.mem_get_info(self.rt.device)
        pages = int(free * fraction) // max(per_page, 1)
        # no request can use more than max_context tokens: more pages than that per slot are never touched
        pages = min(pages, max_requests * ((max_context + page_size - 1) // page_size))
        if pages < 1:
            raise RuntimeError("no memory is left for the cache")
        return pages

    # ---- requests -----------------------------------------------------------
    def admit(self, rid: Hashable) -> int:
        slot = self.manager.admit(rid)
        self.storage.clear_slot(slot)
        return slot

    def release(self, rid: Hashable):
        self.manager.release(rid)

    def has(self, rid: Hashable) -> bool:
        return self.manager.has(rid)

    def n_tokens(self, rid: Hashable) -> int:
        return self.manager.n_tokens(rid)

    def warm_up(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """Capture the graphs now instead of at the first step of each size (a capture takes as long as a few
        hundred steps): the decode steps of the given batch sizes, or, if none is given, of all sizes and the
        steps with prompt portions of every row count as well.  Only while no request is live; returns the
        batch sizes captured (and the row counts, negated)."""
        if self.graphs is None or self.manager.n_live:
            return []
        done = []
        for bucket in self.graphs.buckets:
            if bucket in self.graphs.captured or (batch_sizes is not None and not any(
                    self.graphs.bucket_for(min(b, self.graphs.buckets[-1])) == bucket for b in batch_sizes)):
                continue
            rids = [("warm-up", i) for i in range(bucket)]
            wants = {rid: 1 for rid in rids}
            for rid in rids:
                self.admit(rid)
            try:
                if self.manager.can_reserve(wants):
                    self.manager.reserve(wants)
                    self.graphs.run([StepEntry(rid, [0], [0]) for rid in rids])
                    done.append(bucket)
            finally:
                for rid in rids:
                    self.release(rid)
        if self.portion_graphs is not None and batch_sizes is None:
            # the steps with prompt portions too, for every row count and every number of requests that may bring
            # attention tiles: stand-in requests of two tokens each and one that takes the rest of the rows
            pg = self.portion_graphs
            for rows in pg.buckets:
                n = min(rows, pg.max_context - 1)
                if pg.bucket_for(n) != rows:
                    continue
                for k, tile_pad in enumerate(pg.tile_pads):
                    n_small = 0 if k == 0 else pg.tile_pads[k - 1]       # more requests than the pad below holds
                    if tile_pad in pg.captured.get(rows, {}) or n_small + 1 >= pg.n_requests or n - 2 * n_small < 2:
                        continue
                    counts = [2] * n_small + [n - 2 * n_small]
                    rids = [("warm-up", "rows", rows, i) for i in range(len(counts))]
                    wants = dict(zip(rids, counts))
                    for rid in rids:
                        self.admit(rid)
                    try:
                        if self.manager.can_reserve(wants):
                            self.manager.reserve(wants)
                            pg.run([StepEntry(rid, [0] * c, [c - 1] if i + 1 == len(rids) else [])
                                    for i, (rid, c) in enumerate(zip(rids, counts))])
                            if -rows not in done:
                                done.append(-rows)
                    finally:
                        for rid in rids:
                            self.release(rid)
        return done

    # ---- the step -----------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry], fixed_pages: Optional[Sequence[int]] = None) -> StepContext:
        """Reserve pages for all entries (all or nothing: OutOfPages leaves the cache untouched) and
        build the step's description."""
        wants = {}
        for e in entries:
            if e.rid in wants:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            wants[e.rid] = len(e.tokens)
        self.manager.reserve(wants)
        return build_context(entries, self.manager, self.storage, self.spec.vocab_size, self.spec.max_positions,
                             self.rt.device, fixed_pages)

    def commit(self, entries: Sequence[StepEntry]):
        for e in entries:
            self.manager.commit(e.rid, len(e.tokens))
        self.steps_run += 1

    def _decode_graph_takes(self, entries: Sequence[StepEntry]) -> bool:
        return self.graphs is not None and all(len(e.tokens) == 1 for e in entries) \
            and all(self.manager.n_tokens(e.rid) < self.graphs.max_context for e in entries)

    def takes_carried_tokens(self, entries: Sequence[StepEntry]) -> bool:
        """Whether :meth:`step` can run these entries while some of their token ids are still on the device:
        replayed steps can (their description is completed on the device)."""
        return self._decode_graph_takes(entries) or \
            (self.portion_graphs is not None and self.portion_graphs.takes(entries))

    def step(self, entries: Sequence[StepEntry], own_output: bool = True, carry=None) -> torch.Tensor:
        """float32 logits [number of wanted places, vocab], in the order of entries and of ``want``.

        ``own_output=False`` may return a view of a buffer that the next step overwrites (a replayed
        graph writes to fixed memory); the caller must be done with it before it steps again.
        ``carry`` = (int32 token ids on the device, for every entry its place among them or -1): an entry with a
        place brings one token whose id is still on the device, sampled by the step before; the id in the entry
        is a stand-in (see :meth:`takes_carried_tokens`).
        """
        if carry is not None:
            if len(carry[1]) != len(entries) or any(s >= carry[0].shape[0] for s in carry[1]):
                raise ValueError("carried tokens: one place per entry, each within the given token ids")
            if any(s >= 0 and len(e.tokens) != 1 for e, s in zip(entries, carry[1])):
                raise ValueError("carried tokens: only an entry of a single token can take it from the device")
            if not self.takes_carried_tokens(entries):
                raise ValueError("only a replayed step can take token ids that are still on the device")
        if self._decode_graph_takes(entries):
            wants = {e.rid: 1 for e in entries}
            if len(wants) != len(entries):
                raise ValueError("a request appears twice in one step")
            self.manager.reserve(wants)
            logits = self.graphs.run(entries, carry)
            if own_output:
                logits = logits.clone()
        elif self.portion_graphs is not None and self.portion_graphs.takes(entries):
            wants = {e.rid: len(e.tokens) for e in entries}
            if len(wants) != len(entries):
                raise ValueError("a request appears twice in one step")
            self.manager.reserve(wants)
            logits = self.portion_graphs.run(entries, carry)
            if own_output:
                logits = logits.clone()
        else:
            ctx = self.prepare(entries)
            logits = self.model.forward(ctx)
        self.commit(entries)
        return logits
