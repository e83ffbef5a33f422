"""Host-side book-keeping of the cache: pages, block tables, state slots.

The reference keeps one pool of fixed-size blocks, a per-request table from
block number to block id, and frees a request's blocks when it finishes
(inferrs-models/src/kv_cache.rs:80-139 pool with a FIFO free list, :154-222
table; inferrs/src/engine.rs:746-748 release).  Its store holds only the layers
that see all keys; layers with other needs keep private state inside the model
(inferrs-models/src/config.rs:774-838).

Here the cache is a list of *groups*.  A group is a set of caches (one per
schedule entry that writes keys and values) with the same needs: the same
number of key/value heads, head size and visibility (all keys, or a window).
Each group has a page pool and a block table per request of its own; a window
group gives pages back as soon as the window has passed them.  Beside the
pages there are *state slots*: one slot per live request, the index into
per-request tensors of fixed size (sampler state, and the state of mixers that
keep one).

The book itself is kept by native code (``csrc/host_runtime.cpp``, built with the C++ compiler at first
use like the kernels): this module is its Python front and turns its answers into exceptions.  A model
of the same book in plain Python lives beside the tests and is compared with it call for call.

Nothing here touches the device; :mod:`inferrs_b200.cache.storage` owns the
tensors that the ids point into.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

from ..csrc.build import load_library

RELEASED = -1  # block-table entry of a page that was given back (a window passed it)


class CacheError(RuntimeError):
    """Misuse of the cache manager (unknown request, double free, ...)."""


class OutOfPages(CacheError):
    """Not enough free pages (or no free state slot) for what was asked; nothing was changed."""


@dataclass(frozen=True)
class GroupLayout:
    """What the manager needs to know of a group: which keys stay visible."""

    name: str
    window: Optional[int] = None  # None: all keys; w: a query at i sees keys j with i - w < j <= i


_ERR_UNKNOWN_REQUEST, _ERR_ALREADY_LIVE, _ERR_NO_SLOT, _ERR_OUT_OF_PAGES = -1, -2, -3, -4
_ERR_BAD_COUNT, _ERR_BEYOND_RESERVED, _ERR_DOUBLE_FREE, _ERR_ARGUMENT = -5, -6, -7, -8
ERR_TOKEN, ERR_POSITIONS, ERR_TABLE_WIDTH = -9, -10, -11   # ibh_describe_decode's own refusals

_LIB = None


def host_library():
    """The native host runtime with its argument types set."""
    global _LIB
    if _LIB is None:
        lib = load_library("host_runtime")
        i, p, l = ctypes.c_int, ctypes.c_void_p, ctypes.c_int64
        lib.ibh_cache_new.argtypes = [i, p, p, i, i]
        lib.ibh_cache_new.restype = p
        lib.ibh_cache_delete.argtypes = [p]
        lib.ibh_cache_delete.restype = None
        lib.ibh_sched_new.argtypes = [p, i, i, i, i, p, i]
        lib.ibh_sched_new.restype = p
        lib.ibh_sched_delete.argtypes = [p]
        lib.ibh_sched_delete.restype = None
        for name, args in {
            "ibh_cache_admit": [p, l], "ibh_cache_has": [p, l], "ibh_cache_n_live": [p],
            "ibh_cache_n_free_slots": [p], "ibh_cache_n_free_pages": [p, i], "ibh_cache_slot": [p, l],
            "ibh_cache_n_tokens": [p, l], "ibh_cache_block_table": [p, l, i, p, i],
            "ibh_cache_pages_needed": [p, l, i, p], "ibh_cache_can_reserve": [p, i, p, p],
            "ibh_cache_reserve": [p, i, p, p], "ibh_cache_commit": [p, l, i], "ibh_cache_release": [p, l],
            "ibh_cache_check": [p, ctypes.c_char_p, i],
            "ibh_cache_fit_in_order": [p, i, p, p, p],
            "ibh_describe_decode": [p, i, p, p, i, p, i, i, p, i, p],
            "ibh_describe_step": [p, i, p, p, p, p, p, i, i, i, p, i, p, p, i, i, i, p, i, p],
            "ibh_sched_add": [p, l, i, i, i, p, i], "ibh_sched_abort": [p, l],
            "ibh_sched_plan": [p, i, i, p, p, p, p, p, p, p, p, p],
            "ibh_sched_advance": [p, i, p, p, p], "ibh_sched_deliver": [p, i, p, p, p],
            "ibh_sched_counts": [p, l, p], "ibh_sched_n_waiting": [p], "ibh_sched_n_running": [p],
            "ibh_sched_n_preemptions": [p],
        }.items():
            f = getattr(lib, name)
            f.argtypes = args
            f.restype = i
        _LIB = lib
    return _LIB


class _PoolView:
    """What callers read of one group's pool: its size and how many pages are free."""

    def __init__(self, manager: "CacheManager", group: int, n_pages: int):
        self._m, self._g, self.n_pages = manager, group, n_pages

    @property
    def n_free(self) -> int:
        return self._m._lib.ibh_cache_n_free_pages(self._m._h, self._g)


class CacheManager:
    """Pages of every group and state slots for up to ``max_requests`` live requests.

    A step goes: :meth:`reserve` for every request in it (all or nothing),
    run the kernels, :meth:`commit`.  :meth:`release` ends a request.
    """

    def __init__(self, groups: Sequence[GroupLayout], page_size: int, n_pages: Sequence[int], max_requests: int):
        if page_size <= 0:
            raise CacheError(f"page_size must be positive, got {page_size}")
        if len(n_pages) != len(groups):
            raise CacheError("one page count per group is needed")
        if not groups:
            raise CacheError("at least one group is needed")
        if max_requests <= 0:
            raise CacheError(f"max_requests must be positive, got {max_requests}")
        for g in groups:
            if g.window is not None and g.window <= 0:
                raise CacheError(f"group {g.name}: window must be positive, got {g.window}")
        for n in n_pages:
            if n <= 0:
                raise CacheError(f"a page pool needs at least one page, got {n}")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self._lib = host_library()
        windows = (ctypes.c_int * len(groups))(*[-1 if g.window is None else g.window for g in groups])
        counts = (ctypes.c_int * len(groups))(*[int(n) for n in n_pages])
        self._h = self._lib.ibh_cache_new(len(groups), windows, counts, page_size, max_requests)
        if not self._h:
            raise CacheError("the native cache manager refused these sizes")
        self.pools = [_PoolView(self, g, int(n)) for g, n in enumerate(n_pages)]
        self._handles: Dict[Hashable, int] = {}   # request id -> the number that native code knows it by
        self._next_handle = 0
        self._scratch = (ctypes.c_int * 256)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ibh_cache_delete(h)

    # ---- requests and slots -------------------------------------------------
    def _handle(self, rid: Hashable) -> int:
        try:
            return self._handles[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def handle(self, rid: Hashable) -> int:
        """The number by which native code knows a live request (for calls that pass many at once)."""
        return self._handle(rid)

    def has(self, rid: Hashable) -> bool:
        return rid in self._handles

    # the native scheduler admits and releases requests in the native book itself; the front follows
    def new_handle(self) -> int:
        """A number that no request has had yet (the native scheduler knows a request by it from its arrival)."""
        self._next_handle += 1
        return self._next_handle - 1

    def adopt(self, rid: Hashable, handle: int):
        """Native code has admitted the request under ``handle``."""
        if rid in self._handles:
            raise CacheError(f"request {rid!r} is already live")
        self._handles[rid] = handle

    def forget(self, rid: Hashable):
        """Native code has released the request."""
        self._handles.pop(rid, None)

    @property
    def n_live(self) -> int:
        return len(self._handles)

    @property
    def n_free_slots(self) -> int:
        return self._lib.ibh_cache_n_free_slots(self._h)

    def admit(self, rid: Hashable) -> int:
        """Give the request a state slot and empty block tables; returns the slot."""
        if rid in self._handles:
            raise CacheError(f"request {rid!r} is already live")
        handle = self._next_handle
        slot = self._lib.ibh_cache_admit(self._h, handle)
        if slot == _ERR_NO_SLOT:
            raise OutOfPages(f"no free state slot ({self.max_requests} requests are live)")
        if slot < 0:
            raise CacheError(f"request {rid!r}: the native cache manager answered {slot}")
        self._next_handle += 1
        self._handles[rid] = handle
        return slot

    def slot(self, rid: Hashable) -> int:
        return self._lib.ibh_cache_slot(self._h, self._handle(rid))

    def n_tokens(self, rid: Hashable) -> int:
        return self._lib.ibh_cache_n_tokens(self._h, self._handle(rid))

    def block_table(self, rid: Hashable, group: int) -> List[int]:
        if not 0 <= group < len(self.groups):
            raise CacheError(f"group {group} does not exist")
        handle = self._handle(rid)
        n = self._lib.ibh_cache_block_table(self._h, handle, group, self._scratch, len(self._scratch))
        if n > len(self._scratch):
            self._scratch = (ctypes.c_int * (2 * n))()
            n = self._lib.ibh_cache_block_table(self._h, handle, group, self._scratch, len(self._scratch))
        return self._scratch[:n]

    # ---- pages --------------------------------------------------------------
    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages that each group has to take so that ``n_new`` more tokens fit."""
        out = (ctypes.c_int * len(self.groups))()
        self._lib.ibh_cache_pages_needed(self._h, self._handle(rid), int(n_new), out)
        return list(out)

    def _arrays(self, wants: Dict[Hashable, int]):
        n = len(wants)
        rids = (ctypes.c_int64 * n)(*[self._handle(rid) for rid in wants])
        counts = (ctypes.c_int * n)(*[int(v) for v in wants.values()])
        return n, rids, counts

    def can_reserve(self, wants: Dict[Hashable, int]) -> bool:
        n, rids, counts = self._arrays(wants)
        return self._lib.ibh_cache_can_reserve(self._h, n, rids, counts) == 1

    def fit_in_order(self, rids: Sequence[Hashable], n_new: Sequence[int], free: List[int]) -> int:
        """For a scheduler that walks its requests in order: ``free[g]`` pages of every group are still
        unspoken for; request ``rids[i]`` would take the pages for ``n_new[i]`` more tokens.  Subtracts what each
        one needs from ``free`` (in place) as long as it fits and stops at the first that does not; returns
        how many fitted.  Nothing is taken from the pools."""
        n = len(rids)
        handles = (ctypes.c_int64 * n)(*[self._handle(rid) for rid in rids])
        counts = (ctypes.c_int * n)(*n_new)
        left = (ctypes.c_int * len(self.groups))(*free)
        k = self._lib.ibh_cache_fit_in_order(self._h, n, handles, counts, left)
        if k < 0:
            raise CacheError(f"fit_in_order: the native cache manager answered {k}")
        free[:] = list(left)
        return k

    def reserve(self, wants: Dict[Hashable, int]):
        """Take the pages for ``wants[rid]`` more tokens of every request named, or raise
        OutOfPages and change nothing."""
        for rid, n_new in wants.items():
            if n_new <= 0:
                raise CacheError(f"request {rid!r}: a step must bring at least one token, got {n_new}")
        n, rids, counts = self._arrays(wants)
        code = self._lib.ibh_cache_reserve(self._h, n, rids, counts)
        if code == _ERR_OUT_OF_PAGES:
            need = [sum(self.pages_needed(rid, k)[g] for rid, k in wants.items()) for g in range(len(self.groups))]
            raise OutOfPages("pages wanted per group " + str(need) + ", free " + str([p.n_free for p in self.pools]))
        if code != 0:
            raise CacheError(f"reserve: the native cache manager answered {code}")

    def commit(self, rid: Hashable, n_new: int):
        """The step wrote ``n_new`` tokens; give back the pages that every later query's window has passed."""
        code = self._lib.ibh_cache_commit(self._h, self._handle(rid), int(n_new))
        if code == _ERR_BEYOND_RESERVED:
            raise CacheError(f"request {rid!r}: commit of {n_new} tokens beyond those reserved")
        if code != 0:
            raise CacheError(f"commit: the native cache manager answered {code}")

    def release(self, rid: Hashable):
        """The request is over: all its pages and its slot are free again."""
        code = self._lib.ibh_cache_release(self._h, self._handle(rid))
        del self._handles[rid]
        if code != 0:
            raise CacheError(f"release: the native cache manager answered {code}")

    # ---- checks -------------------------------------------------------------
    def check_invariants(self):
        """No page lost, none held by two requests, free list and tables disjoint."""
        msg = ctypes.create_string_buffer(256)
        if self._lib.ibh_cache_check(self._h, msg, 256) != 0:
            raise CacheError(msg.value.decode())
        if self._lib.ibh_cache_n_live(self._h) != len(self._handles):
            raise CacheError("the front and the native book disagree on the live requests")

    def describe_decode(self, rids: Sequence[Hashable], tokens: Sequence[int], bucket: int,
                        fixed_pages: Sequence[int], vocab_size: int, max_positions: int, out_ptr: int, cap: int):
        """Write the description of a step of single tokens, padded to ``bucket`` requests, to ``cap`` int32
        at ``out_ptr`` (host memory), in the layout of :func:`inferrs_b200.engine.batch.build_context`.
        Returns (numbers written, 0) or (a negative refusal, index of the entry it is about)."""
        n = len(rids)
        handles = (ctypes.c_int64 * n)(*[self._handle(rid) for rid in rids])
        toks = (ctypes.c_int * n)(*tokens)
        pages = (ctypes.c_int * len(self.groups))(*fixed_pages)
        bad = ctypes.c_int(0)
        code = self._lib.ibh_describe_decode(self._h, n, handles, toks, bucket, pages, vocab_size, max_positions,
                                             out_ptr, cap, ctypes.byref(bad))
        return code, bad.value

    def describe_step(self, rids: Sequence[Hashable], tokens: Sequence[Sequence[int]], wants: Sequence[Sequence[int]],
                      pad_rows: int, pad_requests: int, pad_wanted: int, fixed_pages: Sequence[int],
                      tile_sizes: Sequence[tuple], tile_pad: int, vocab_size: int, max_positions: int, out_ptr: int,
                      cap: int):
        """The same for a step of any portions, padded to ``pad_rows`` rows, ``pad_requests`` requests and
        ``pad_wanted`` wanted places, with a tile list of fixed length for every (tokens per tile, portions only)
        pair (room for ``pad_rows // tokens + tile_pad`` tiles): the layout of ``build_context(..., pad_rows=...)``.  Returns (numbers written, 0) or (a negative
        refusal, index of the entry it is about)."""
        import numpy as np
        n = len(rids)
        handles = (ctypes.c_int64 * n)(*[self._handle(rid) for rid in rids])
        n_tok = (ctypes.c_int * n)(*[len(t) for t in tokens])
        n_want = (ctypes.c_int * n)(*[len(w) for w in wants])
        flat = np.fromiter((t for ts in tokens for t in ts), dtype=np.int64)
        if flat.size and (flat.min() < 0 or flat.max() >= vocab_size):
            return ERR_TOKEN, 0
        flat = flat.astype(np.int32)
        flat_w = np.fromiter((w for ws in wants for w in ws), dtype=np.int64).astype(np.int32)
        pages = (ctypes.c_int * len(self.groups))(*fixed_pages)
        k = len(tile_sizes)
        tile_tokens = (ctypes.c_int * max(k, 1))(*[t for t, _ in tile_sizes])
        tile_portions = (ctypes.c_int * max(k, 1))(*[int(bool(po)) for _, po in tile_sizes])
        bad = ctypes.c_int(0)
        code = self._lib.ibh_describe_step(self._h, n, handles, n_tok, flat.ctypes.data, n_want, flat_w.ctypes.data,
                                           pad_rows, pad_requests, pad_wanted, pages, k, tile_tokens, tile_portions,
                                           tile_pad, vocab_size, max_positions, out_ptr, cap, ctypes.byref(bad))
        return code, bad.value
