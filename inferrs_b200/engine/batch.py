"""One step's batch: which tokens of which requests run, and what the kernels need to know of them.

The reference runs one sequence per forward pass, either its whole prompt or
one decoded token (inferrs/src/engine.rs:2074-2147), and resolves cache slots
on the host per pass (inferrs-models/src/models/attention_utils.rs:252-283).
Here a step is a flat list of rows: every request contributes its next tokens,
a portion of a prompt or a single decoded token, and the rows of one request
stand together in order.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    """Device tensors (int32) and host numbers that describe a step to the parts.

    token_ids [N]      the rows' token ids
    positions [N]      each row's position within its request
    row_request [N]    each row's index into this step's requests
    q_start [R+1]      rows q_start[r] .. q_start[r+1]-1 belong to request r
    kv_len [R]         tokens of request r in the cache once this step's keys are written
    slots [R]          state slot of request r
    logit_rows [W]     rows whose logits are returned, in the order of entries and of ``want``
    block_tables[g]    [R, max_pages_g] page ids of request r in cache group g (-1: given back)
    """

    token_ids: torch.Tensor
    positions: torch.Tensor
    row_request: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    block_tables: List[torch.Tensor]
    storage: CacheStorage
    n_rows: int
    n_requests: int
    q_lens: List[int]
    kv_lens: List[int]
    slot_list: List[int]
    max_q_len: int
    max_kv_len: int
    extra: dict = field(default_factory=dict)

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1

    def attention_tiles(self, tokens_per_tile: int, portions_only: bool = False):
        """(tile_req, tile_row0, n_tiles): the step's rows cut into tiles of at most ``tokens_per_tile``
        tokens of one request each; with ``portions_only`` without the requests that bring a single token
        (:meth:`single_rows` has those).  Made once per step and tile size, on first use."""
        key = ("attention_tiles", tokens_per_tile, portions_only)
        if key not in self.extra:
            tiles = sorted_tiles(self.q_lens, [k - n for k, n in zip(self.kv_lens, self.q_lens)], tokens_per_tile,
                                 portions_only)
            both = torch.from_numpy(np.asarray([[t[1] for t in tiles], [t[2] for t in tiles]],
                                               dtype=np.int32).reshape(2, -1)).to(self.token_ids.device)
            self.extra[key] = (both[0], both[1], len(tiles))
        return self.extra[key]

    def single_rows(self):
        """(rows, requests, count) of the requests that bring a single token to the step."""
        key = "single_rows"
        if key not in self.extra:
            rows, reqs, at = [], [], 0
            for r, n in enumerate(self.q_lens):
                if n == 1:
                    rows.append(at)
                    reqs.append(r)
                at += n
            both = torch.from_numpy(np.asarray([rows, reqs], dtype=np.int32).reshape(2, -1)).to(self.token_ids.device)
            self.extra[key] = (both[0], both[1], len(rows))
        return self.extra[key]


class BatchError(ValueError):
    pass


def sorted_tiles(q_lens: Sequence[int], starts: Sequence[int], tokens_per_tile: int, portions_only: bool):
    """The step's rows cut into tiles of at most ``tokens_per_tile`` tokens of one request each, as
    (position of the tile's last token, request, first row); ``starts[r]`` is the position of request r's first token
    of the step.  The tile that sees the fewest keys comes first: the attention kernels start at the end of the list,
    with the longest tile, so that the grid's tail is short."""
    tiles, at = [], 0
    for r, n in enumerate(q_lens):
        if not (portions_only and n == 1):
            for s in range(0, n, tokens_per_tile):
                tiles.append((starts[r] + min(s + tokens_per_tile, n) - 1, r, at + s))
        at += n
    tiles.sort(key=lambda t: t[0])      # stable: tiles that see as many keys keep their order
    return tiles


def build_context(entries: Sequence[StepEntry], manager: CacheManager, storage: CacheStorage, vocab_size: int,
                  max_positions: int, device: torch.device, fixed_pages: Optional[Sequence[int]] = None,
                  pad_to: Optional[int] = None, into: Optional[torch.Tensor] = None,
                  pad_rows: Optional[int] = None, pad_requests: Optional[int] = None,
                  pad_wanted: Optional[int] = None, tile_sizes: Sequence[int] = (),
                  tile_pad: Optional[int] = None) -> StepContext:
    """Check the entries and lay their rows out.  Pages must already be reserved in ``manager``.

    ``fixed_pages[g]`` pads group g's block table to that many columns, ``pad_to`` pads a step of
    single tokens to that many requests, and ``into`` is a device buffer that receives the data:
    together they give a step whose shapes and addresses do not change, which a replayed CUDA
    graph needs.  A padding request has one token at position 0, no pages and the state slot after
    the last real one: it writes nothing to the cache or to a live request's state, and its
    output is not used.

    ``pad_rows`` does the same for a step of any portions: the rows are padded to ``pad_rows`` (the
    added rows belong to one padding request without pages), the requests to ``pad_requests``, the
    wanted places to ``pad_wanted`` (row 0 stands in), and for every (number of tokens, portions
    only) pair in ``tile_sizes`` the list of attention tiles is laid out with a fixed length
    (``pad_rows // tokens + tile_pad``; ``tile_pad``, the most requests that may bring tiles, is
    ``pad_requests`` if not given), the tiles at its end in the order of :func:`sorted_tiles` and -1
    marking the places before them that hold no tile; the list of the requests that bring a single
    token has ``pad_requests`` places.
    """
    if not entries:
        raise BatchError("a step needs at least one entry")
    seen = set()
    id_parts, pos_parts, req_parts = [], [], []
    q_start = [0]
    kv_lens, slots, logit_rows, q_lens = [], [], [], []
    for r, e in enumerate(entries):
        if e.rid in seen:
            raise BatchError(f"request {e.rid!r} appears twice in one step")
        seen.add(e.rid)
        try:
            toks = np.asarray(e.tokens)
        except (TypeError, ValueError):
            raise BatchError(f"request {e.rid!r}: the tokens are not a list of integers") from None
        if toks.ndim != 1 or toks.size == 0:
            raise BatchError(f"request {e.rid!r}: a step must bring at least one token")
        if toks.dtype.kind not in "iu":
            raise BatchError(f"request {e.rid!r}: token ids must be integers, got {toks.dtype}")
        lo, hi = int(toks.min()), int(toks.max())
        if lo < 0 or hi >= vocab_size:
            bad = lo if lo < 0 else hi
            raise BatchError(f"request {e.rid!r}: token id {bad!r} is outside the vocabulary of {vocab_size}")
        n_tok = int(toks.size)
        held = manager.n_tokens(e.rid)
        if held + n_tok > max_positions:
            raise BatchError(f"request {e.rid!r}: {held} + {n_tok} tokens exceed the model's "
                             f"{max_positions} positions")
        for w in e.want:
            if not 0 <= int(w) < n_tok:
                raise BatchError(f"request {e.rid!r}: wanted place {w} is outside its {n_tok} tokens")
            logit_rows.append(q_start[-1] + int(w))
        id_parts.append(toks.astype(np.int32, copy=False))
        pos_parts.append(np.arange(held, held + n_tok, dtype=np.int32))
        req_parts.append(np.full(n_tok, r, dtype=np.int32))
        q_start.append(q_start[-1] + n_tok)
        q_lens.append(n_tok)
        kv_lens.append(held + n_tok)
        slots.append(manager.slot(e.rid))
    ids = np.concatenate(id_parts).tolist() if pad_to is not None else None
    positions = np.concatenate(pos_parts).tolist() if pad_to is not None else None
    row_request = np.concatenate(req_parts).tolist() if pad_to is not None else None
    n_real = len(entries)
    tiles_fixed = {}
    if pad_rows is not None:
        if pad_to is not None or pad_requests is None or pad_wanted is None:
            raise BatchError("pad_rows needs pad_requests and pad_wanted, and excludes pad_to")
        n_rows_real = q_start[-1]
        if n_rows_real > pad_rows or n_real + 1 > pad_requests or len(logit_rows) > pad_wanted:
            raise BatchError(f"{n_rows_real} rows, {n_real} requests and {len(logit_rows)} wanted places do not fit "
                             f"the fixed step of {pad_rows} rows, {pad_requests} requests, {pad_wanted} places")
        for tpt, portions_only in tile_sizes:   # the tiles of the real requests; the padding request gets none
            t_max = pad_rows // tpt + (pad_requests if tile_pad is None else tile_pad)
            req = np.full(t_max, -1, dtype=np.int32)
            row0 = np.zeros(t_max, dtype=np.int32)
            tiles = sorted_tiles(q_lens[:n_real], [k - n for k, n in zip(kv_lens, q_lens)], tpt, portions_only)
            if len(tiles) > t_max:
                raise BatchError(f"{len(tiles)} attention tiles of {tpt} tokens do not fit the fixed list of {t_max}")
            first = t_max - len(tiles)
            for k, (_, r, r0) in enumerate(tiles):
                req[first + k], row0[first + k] = r, r0
            tiles_fixed[(tpt, portions_only)] = (req, row0, t_max)
        single = np.full((2, pad_requests), -1, dtype=np.int32)   # rows and requests of the single tokens
        k = 0
        for r in range(n_real):
            if q_lens[r] == 1:
                single[0, k], single[1, k] = q_start[r], r
                k += 1
        extra_rows = pad_rows - n_rows_real
        id_parts.append(np.zeros(extra_rows, dtype=np.int32))
        pos_parts.append(np.zeros(extra_rows, dtype=np.int32))
        req_parts.append(np.full(extra_rows, n_real, dtype=np.int32))
        for r in range(n_real, pad_requests):
            k = extra_rows if r == n_real else 0
            q_start.append(q_start[-1] + k)
            q_lens.append(k)
            kv_lens.append(max(k, 1))
            slots.append(manager.max_requests)   # the slot that no request ever gets
        wanted = list(logit_rows)
        logit_rows = logit_rows + [0] * (pad_wanted - len(logit_rows))
    if pad_to is not None:
        if any(q != 1 for q in q_lens) or len(entries) > pad_to:
            raise BatchError("only steps of single tokens, no more than pad_to of them, can be padded")
        for r in range(len(entries), pad_to):
            ids.append(0)
            positions.append(0)
            row_request.append(r)
            q_start.append(q_start[-1] + 1)
            q_lens.append(1)
            kv_lens.append(1)
            slots.append(manager.max_requests)   # the slot that no request ever gets
        wanted = list(logit_rows)
        logit_rows = list(range(pad_to))  # fixed shape: every row's logits are made, the caller picks
    elif pad_rows is None:
        wanted = None
    n, nreq = q_start[-1], len(q_lens)
    tables = []
    for g in range(len(manager.groups)):
        rows = [manager.block_table(e.rid, g) for e in entries]
        width = max(1, max(len(t) for t in rows))
        if fixed_pages is not None:
            if width > fixed_pages[g]:
                raise BatchError(f"group {g}: a block table of {width} pages exceeds the fixed {fixed_pages[g]}")
            width = fixed_pages[g]
        arr = np.full((nreq, width), -1, dtype=np.int32)
        for r, t in enumerate(rows):  # padding requests keep -1 everywhere
            arr[r, :len(t)] = t
        tables.append(arr)
    # one host buffer, one copy
    if pad_to is not None:   # a short step of single tokens: plain lists, padded above
        first = [np.asarray(ids, dtype=np.int32), np.asarray(positions, dtype=np.int32),
                 np.asarray(row_request, dtype=np.int32)]
    else:
        first = [np.concatenate(id_parts), np.concatenate(pos_parts), np.concatenate(req_parts)]
    parts = first + [np.asarray(q_start, dtype=np.int32),
             np.asarray(kv_lens, dtype=np.int32), np.asarray(slots, dtype=np.int32),
             np.asarray(logit_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables]
    tile_at = {}
    for key, (req, row0, t_max) in tiles_fixed.items():
        tile_at[key] = len(parts)
        parts += [req, row0]
    single_at = None
    if pad_rows is not None:
        single_at = len(parts)
        parts += [single[0], single[1]]
    sizes = [p.size for p in parts]
    # every part starts on a 16-byte boundary, which vector loads and bulk copies need
    offsets, total = [], 0
    for s in sizes:
        offsets.append(total)
        total += (s + 3) // 4 * 4
    host = np.zeros(max(total, 4), dtype=np.int32)
    for p, o in zip(parts, offsets):
        host[o:o + p.size] = p
    if into is not None:
        if into.numel() < host.size:
            raise BatchError(f"the fixed step buffer holds {into.numel()} numbers, {host.size} are needed")
        dev = into
        dev[:host.size].copy_(torch.from_numpy(host))
    else:
        dev = torch.from_numpy(host).to(device)
    views = [dev[o:o + s] for o, s in zip(offsets, sizes)]
    extra = {"n_real": n_real, "wanted": wanted, "host": host}
    for key, at in tile_at.items():
        extra[("attention_tiles",) + key] = (views[at], views[at + 1], tiles_fixed[key][2])
    if single_at is not None:
        extra["single_rows"] = (views[single_at], views[single_at + 1], pad_requests)
    return StepContext(
        token_ids=views[0], positions=views[1], row_request=views[2], q_start=views[3], kv_len=views[4],
        slots=views[5], logit_rows=views[6],
        block_tables=[views[7 + g].view(nreq, tables[g].shape[1]) for g in range(len(tables))],
        storage=storage, n_rows=n, n_requests=nreq, q_lens=q_lens, kv_lens=kv_lens, slot_list=slots,
        max_q_len=max(q_lens) if pad_rows is None else max(2, max(q_lens)), max_kv_len=max(kv_lens), extra=extra)
