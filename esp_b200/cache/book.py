"""Host-side bookkeeping of the cache: which slot a sequence holds, how long it
is, and which pages of each layer group's pool carry its keys and values.

Nothing here touches a device.  A *slot* is a sequence's handle for the time it
lives; a *page* holds PAGE consecutive positions of one sequence (for every
layer of its group).  Layers with the same needs form a group with a pool of
its own: a group of full-attention layers keeps every position, a group of
windowed layers gives pages back once the window has passed them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import CacheFull, InvalidRequest

PAGE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


class FreeList:
    """Hands out integers 0..n-1; an id is held by one owner at a time.  Ids
    that were given back last are handed out first, so a finished sequence's
    slot and pages are the next ones used."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))
        self._held = set()

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self, count: int = 1) -> list:
        if count > len(self._free):
            raise CacheFull(f"no free {self.what}: asked for {count}, {len(self._free)} of {self.n} left")
        got = [self._free.pop() for _ in range(count)]
        self._held.update(got)
        return got

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if i not in self._held:
                raise InvalidRequest(f"{self.what} {i} is not held (given back twice, or never taken)")
        if len(set(ids)) != len(ids):
            raise InvalidRequest(f"a {self.what} is named twice in one release")
        for i in ids:
            self._held.discard(i)
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return i in self._held


@dataclass(frozen=True)
class KvLayout:
    """What a layer asks of the cache; layers with equal layouts share a group."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: keep every position


class GroupBook:
    """Pages of one layer group.  ``tables[slot][i]`` is the page that holds
    positions [i*PAGE, (i+1)*PAGE) of the slot's sequence, or -1 when no page
    is held for them (not yet written, or already behind the window)."""

    def __init__(self, layout: KvLayout, n_pages: int):
        self.layout = layout
        self.pool = FreeList(n_pages, "cache page")
        self.tables: dict = {}

    def first_needed(self, length: int) -> int:
        """First position that a query at position ``length`` can still see."""
        if self.layout.window is None:
            return 0
        return max(0, length - self.layout.window + 1)

    def missing(self, slot: int, old_len: int, new_len: int) -> list:
        """Page indices that a step taking the slot from old_len to new_len
        needs and does not hold yet."""
        table = self.tables.get(slot, [])
        hi = pages_for(new_len)
        if self.layout.window is None:
            # nothing is ever given back before the slot closes: the table has no gaps
            return list(range(len(table), hi)) if hi > len(table) else []
        lo = self.first_needed(old_len) // PAGE
        return [i for i in range(lo, hi) if i >= len(table) or table[i] < 0]

    def reserve(self, slot: int, old_len: int, new_len: int) -> tuple:
        """Takes the pages the step needs.  Returns what ``cancel`` needs to undo it."""
        need = self.missing(slot, old_len, new_len)
        got = self.pool.take(len(need))
        table = self.tables.setdefault(slot, [])
        before = len(table)
        hi = pages_for(new_len)
        while len(table) < hi:
            table.append(-1)
        for i, page in zip(need, got):
            table[i] = page
        return slot, before, need

    def cancel(self, receipt: tuple) -> None:
        """Gives back the pages of a reservation whose step did not run to its end."""
        slot, before, need = receipt
        table = self.tables.get(slot)
        if table is None:
            return
        self.pool.give_back([table[i] for i in need])
        for i in need:
            table[i] = -1
        del table[before:]

    def trim(self, slot: int, length: int) -> None:
        """Give back pages that no later query of the slot can see."""
        table = self.tables.get(slot)
        if not table or self.layout.window is None:
            return
        keep_from = self.first_needed(length) // PAGE
        gone = [p for p in table[:keep_from] if p >= 0]
        if gone:
            self.pool.give_back(gone)
            for i in range(min(keep_from, len(table))):
                table[i] = -1

    def release(self, slot: int) -> None:
        table = self.tables.pop(slot, [])
        self.pool.give_back([p for p in table if p >= 0])

    def table_rows(self, slots, stride: int) -> list:
        """One row of ``stride`` page ids per slot (-1 padded) for the device."""
        rows = []
        for s in slots:
            t = self.tables.get(s, [])
            if len(t) > stride:
                raise InvalidRequest(f"slot {s} holds {len(t)} pages, more than the table stride {stride}")
            rows.append(t + [-1] * (stride - len(t)))
        return rows


class CacheBook:
    """Slots, lengths and the page tables of every group."""

    def __init__(self, layouts: list, max_tokens: int, max_slots: int, max_positions: int):
        if max_tokens <= 0 or max_slots <= 0:
            raise InvalidRequest("the cache needs room for at least one token and one slot")
        self.n_pages = pages_for(max_tokens)
        self.max_positions = max_positions
        self.slots = FreeList(max_slots, "cache slot")
        self.groups = [GroupBook(l, self.n_pages) for l in layouts]
        self.lengths: dict = {}

    def open(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        return slot

    def length(self, slot: int) -> int:
        if slot not in self.lengths:
            raise InvalidRequest(f"slot {slot} is not open")
        return self.lengths[slot]

    def check_step(self, growth: dict) -> None:
        """``growth``: slot -> number of new tokens.  Raises without changing
        anything if a sequence would pass the longest position or the pools
        cannot hold the step."""
        for slot, n_new in growth.items():
            old = self.length(slot)
            if n_new <= 0:
                raise InvalidRequest(f"slot {slot}: a step must bring at least one token")
            if old + n_new > self.max_positions:
                raise InvalidRequest(f"slot {slot}: {old} cached + {n_new} new tokens pass the model's "
                                     f"{self.max_positions} positions")
        for g in self.groups:
            need = sum(len(g.missing(s, self.lengths[s], self.lengths[s] + n)) for s, n in growth.items())
            if need > g.pool.available:
                raise CacheFull(f"the step needs {need} more cache pages of {PAGE} tokens, "
                                f"{g.pool.available} of {g.pool.n} are free")

    def reserve(self, growth: dict) -> list:
        """Takes the pages of a step (all of them or, with CacheFull, none).  The
        result goes to ``commit`` once the step has run, or to ``cancel`` if it
        has not."""
        self.check_step(growth)
        receipts = []
        for g in self.groups:
            for slot, n_new in growth.items():
                receipts.append((g, g.reserve(slot, self.lengths[slot], self.lengths[slot] + n_new)))
        return receipts

    def cancel(self, receipts: list) -> None:
        """Undoes ``reserve``: the step failed, its sequences keep their old
        lengths and hold no page more than before."""
        for g, receipt in reversed(receipts):
            g.cancel(receipt)

    def commit(self, growth: dict) -> None:
        for slot, n_new in growth.items():
            self.lengths[slot] += n_new
            for g in self.groups:
                g.trim(slot, self.lengths[slot])

    def close(self, slot: int) -> None:
        if slot not in self.lengths:
            raise InvalidRequest(f"slot {slot} is not open (closed twice?)")
        for g in self.groups:
            g.release(slot)
        del self.lengths[slot]
        self.slots.give_back([slot])

    def live_slots(self) -> list:
        return sorted(self.lengths)
