"""Device memory of the cache: page tensors of every group and per-request state.

The reference allocates, per layer, K and V tensors ``[blocks * block_size,
kv_heads, head_dim]`` (inferrs-models/src/kv_cache.rs:249-270).  Here one
tensor per group holds all its caches,

    [caches in group, 2 (keys, values), pages, kv_heads, page_size, head_dim]

so that one page of one head is a contiguous ``[page_size, head_dim]`` tile.
Writes are plain stores; a page that is used again needs no clearing because a
request never reads beyond the tokens it has written.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .manager import GroupLayout


@dataclass(frozen=True)
class KVNeed:
    """What a mixer asks of the paged cache for one schedule entry."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps for one schedule entry."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheStorage:
    def __init__(self, kv_needs: Dict[int, KVNeed], state_needs: Dict[int, StateNeed], page_size: int,
                 n_pages: int, max_requests: int, dtype: torch.dtype, device: torch.device,
                 n_pages_per_group: Optional[Sequence[int]] = None):
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = device
        # caches with equal needs form a group, in order of first appearance
        keys: List[KVNeed] = []
        self.group_of: Dict[int, int] = {}
        self.index_in_group: Dict[int, int] = {}
        members: List[List[int]] = []
        for cid in sorted(kv_needs):
            need = kv_needs[cid]
            if need not in keys:
                keys.append(need)
                members.append([])
            g = keys.index(need)
            self.group_of[cid] = g
            self.index_in_group[cid] = len(members[g])
            members[g].append(cid)
        self.needs = keys
        self.members = members
        self.layouts = [GroupLayout(name=f"group{g}(heads={k.n_kv_heads},dim={k.head_dim},window={k.window})",
                                    window=k.window) for g, k in enumerate(keys)]
        self.n_pages = list(n_pages_per_group) if n_pages_per_group is not None else [n_pages] * len(keys)
        self.kv: List[torch.Tensor] = []
        for g, k in enumerate(keys):
            self.kv.append(torch.zeros((len(members[g]), 2, self.n_pages[g], k.n_kv_heads, page_size, k.head_dim),
                                       dtype=dtype, device=device))
        # one slot more than there are requests: the requests that only pad a replayed step write their state there
        self.states: Dict[int, torch.Tensor] = {
            cid: torch.zeros((max_requests + 1,) + tuple(need.shape), dtype=need.dtype, device=device)
            for cid, need in state_needs.items()}

    def pages(self, cache_id: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """(key pages, value pages, group index) of one cache; pages are [n_pages, kv_heads, page_size, head_dim]."""
        g = self.group_of[cache_id]
        t = self.kv[g][self.index_in_group[cache_id]]
        return t[0], t[1], g

    def state(self, cache_id: int) -> torch.Tensor:
        return self.states[cache_id]

    def clear_slot(self, slot: int):
        """A new request takes the slot: its fixed-size states start at zero."""
        for t in self.states.values():
            t[slot].zero_()

    def snapshot_states(self) -> Dict[int, torch.Tensor]:
        """Copies of all fixed-size states (for a caller that has to run a step more than once)."""
        return {cid: t.clone() for cid, t in self.states.items()}

    def restore_states(self, saved: Dict[int, torch.Tensor]):
        for cid, t in saved.items():
            self.states[cid].copy_(t)

    def bytes_per_token(self) -> int:
        """Bytes of keys and values that one token adds, over all groups."""
        e = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(self.members[g]) * k.n_kv_heads * k.head_dim * e for g, k in enumerate(self.needs))

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.states.values())
