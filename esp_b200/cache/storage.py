"""Device storage behind the bookkeeping: the key/value pools of every layer
group and the per-sequence state of fixed size."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import InvalidRequest
from .book import PAGE, CacheBook, KvLayout

# words of the engine's own per-sequence state (int64 each)
STATE_RNG = 0          # splitmix64 state of the sequence's sampler
STATE_WORDS = 4        # a row is 32 bytes; the other words are free


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size that a mixer keeps (one per slot)."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one call of a layer sees of the cache."""
    k: Optional[torch.Tensor]          # [pages, nkv, PAGE, hd] of this layer
    v: Optional[torch.Tensor]
    group: Optional[int]               # index of its group (selects the step's page table)
    writes: bool                       # False: it reads another call's keys and values
    state: Optional[torch.Tensor]      # [max_slots, *StateSpec.shape]
    page: int = PAGE


class Cache:
    """``requests``: one (KvLayout or None, StateSpec or None, cache_of or None)
    per schedule entry, in schedule order."""

    def __init__(self, requests: list, max_tokens: int, max_slots: int, max_positions: int, dtype, device):
        self.device = device
        self.dtype = dtype
        layouts, members = [], []
        owner_group = {}
        for idx, (layout, _state, cache_of) in enumerate(requests):
            if cache_of is not None:
                if cache_of >= idx or requests[cache_of][2] is not None:
                    raise InvalidRequest(f"schedule entry {idx} reads the cache of entry {cache_of}, which must be "
                                         f"an earlier entry with a cache of its own")
                continue
            if layout is None:
                continue
            if layout not in layouts:
                layouts.append(layout)
                members.append([])
            g = layouts.index(layout)
            owner_group[idx] = (g, len(members[g]))
            members[g].append(idx)
        self.book = CacheBook(layouts, max_tokens, max_slots, max_positions)
        self.layouts = layouts
        self.members = members
        n_pages = self.book.n_pages
        self.k_pools, self.v_pools = [], []
        for layout, m in zip(layouts, members):
            shape = (len(m), n_pages, layout.num_kv_heads, PAGE, layout.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v_pools.append(torch.zeros(shape, dtype=dtype, device=device))
        self.engine_state = torch.zeros((max_slots, STATE_WORDS), dtype=torch.int64, device=device)
        self.layers = []
        for idx, (layout, state, cache_of) in enumerate(requests):
            st = None
            if state is not None:
                st = torch.zeros((max_slots, *state.shape), dtype=state.dtype, device=device)
            src = cache_of if cache_of is not None else idx
            if src in owner_group:
                g, j = owner_group[src]
                self.layers.append(LayerCache(self.k_pools[g][j], self.v_pools[g][j], g, cache_of is None, st))
            else:
                self.layers.append(LayerCache(None, None, None, False, st))

    # -- slots -----------------------------------------------------------------
    def open(self) -> int:
        slot = self.book.open()
        self.engine_state[slot].zero_()
        for layer in self.layers:
            if layer.state is not None:
                layer.state[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.book.close(slot)

    def max_table_stride(self, slots, growth) -> int:
        """Pages that the longest sequence of the step will hold."""
        longest = max(self.book.length(s) + growth.get(s, 0) for s in slots)
        return max(1, (longest + PAGE - 1) // PAGE)

    def bytes_per_token(self) -> int:
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(m) * l.num_kv_heads * l.head_dim * el for l, m in zip(self.layouts, self.members))
