"""The cache: a slot per live sequence, paged keys and values per storage group, and a
fixed-size per-sequence state area.

Storage groups. Cache entries (one per schedule entry that writes a cache) with the same need
(kind, K/V heads, head size, window) share a group; each group has its own page pool and its
own device storage ``k, v: [entries, pages, kv_heads, PAGE, head_dim]``. A ``full`` group keeps
every key and value of a sequence; a ``window`` group gives pages back once every position in
them is older than the window (positions left of ``length - window`` are never read again).
The reference's analogues are StaticCache (src/transformers/cache_utils.py:1058-1230: storage
allocated once, written in place), HybridCache (:1550-1743: per-layer kinds with their own
shapes) and MambaCache (:1746-1859: fixed-size state per batch row, reset in place).

Sizing. ``max_tokens`` is the most tokens that live sequences hold at one time, each sequence's
count rounded up to a whole page of 64; every group gets ``max_tokens / 64`` pages.

Sequences. ``open()`` gives a slot, ``reserve(slot, n)`` gets the pages for ``n`` more tokens
(or raises CacheFull before anything is launched), ``commit(slot, n)`` advances the length
after the step, ``close(slot)`` gives pages and slot back. Storage is zeroed when it is
allocated and never again: lengths and page lists gate every read. The state area is zeroed for a slot when it is opened.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, StateNeed
from .pool import CacheError, CacheFull, IdPool, SequenceRecord

PAGE = 64

# What a kind of cache entry keeps: for a sequence of `length` tokens, the first position that a later
# query can still see (pages that lie wholly before it go back to the pool after every step).
# ``register_cache_kind`` adds a kind without a change here; the mixer that names it reads accordingly.
CACHE_KINDS = {
    "full": lambda need, length: 0,
    # the next query sits at position >= length and sees keys > position - window
    "window": lambda need, length: max(0, length - need.window + 1),
}


def register_cache_kind(kind: str, first_needed) -> None:
    """``first_needed(need: CacheNeed, length: int) -> int``: the first cached position that queries at
    positions >= length may read."""
    CACHE_KINDS[kind] = first_needed


class StorageGroup:
    def __init__(self, need: CacheNeed, entries: List[int], num_pages: int, dtype: torch.dtype, device):
        if need.kind not in CACHE_KINDS:
            raise ValueError(f"unknown cache kind {need.kind!r} (kinds: {', '.join(sorted(CACHE_KINDS))})")
        if need.kind == "window" and need.window <= 0:
            raise ValueError("a window group needs window > 0")
        self.need = need
        self.entries = list(entries)
        self.index_of = {e: i for i, e in enumerate(self.entries)}
        self.pool = IdPool(num_pages, "cache page")
        shape = (len(self.entries), num_pages, need.kv_heads, PAGE, need.head_dim)
        # zeroed once: kernels multiply masked positions of a page by zero, which must not meet a NaN
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class Cache:
    def __init__(self, needs: Sequence[Tuple[int, Optional[CacheNeed], Optional[StateNeed]]], max_tokens: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None):
        if max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {max_tokens}")
        self.num_pages = (max_tokens + PAGE - 1) // PAGE
        self.max_tokens = self.num_pages * PAGE
        self.dtype, self.device = dtype, torch.device(device)
        by_need: Dict[CacheNeed, List[int]] = {}
        for entry, need, _ in needs:
            if need is not None:
                by_need.setdefault(need, []).append(entry)
        self.groups: List[StorageGroup] = [StorageGroup(n, es, self.num_pages, dtype, self.device)
                                           for n, es in by_need.items()]
        self.group_of_entry: Dict[int, int] = {e: gi for gi, g in enumerate(self.groups) for e in g.entries}
        # a live sequence holds at least one page of every group, so pages bound the slots
        self.max_slots = int(max_slots) if max_slots is not None else max(1, min(self.num_pages, 4096))
        self.slots = IdPool(self.max_slots, "sequence slot")
        self.records: Dict[int, SequenceRecord] = {}
        self.epoch = 0   # counts opened and closed sequences: what was planned for an earlier epoch is stale
        self.state_entries: Dict[int, int] = {}
        self.state: Optional[torch.Tensor] = None
        widths = [(e, s.numel) for e, _, s in needs if s is not None and s.numel > 0]
        self.state_offsets: Dict[int, Tuple[int, int]] = {}
        off = 0
        for e, n in widths:
            self.state_offsets[e] = (off, n)
            off += n
        self.state_width = off
        # the state area exists for every model; for one without stateful mixers it has width 0
        self.state = torch.zeros((self.max_slots, self.state_width), dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        (slot,) = self.slots.take(1)
        self.epoch += 1
        self.records[slot] = SequenceRecord(len(self.groups))
        if self.state_width:
            self.state[slot].zero_()
        return slot

    def _record(self, slot: int) -> SequenceRecord:
        try:
            return self.records[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not open") from None

    def length(self, slot: int) -> int:
        return self._record(slot).length

    def reserve(self, slot: int, n_new: int) -> None:
        """Make sure ``slot`` has pages for ``n_new`` more tokens in every group."""
        rec = self._record(slot)
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        want = (rec.length + n_new + PAGE - 1) // PAGE
        for gi, g in enumerate(self.groups):
            have = len(rec.pages[gi])
            if want > have:
                rec.pages[gi].extend(g.pool.take(want - have))

    def reserve_all(self, plan: Sequence[Tuple[int, int]]) -> None:
        """Reserve for several sequences at once; if the pages do not suffice, nothing is kept."""
        need = [0] * len(self.groups)
        for slot, n_new in plan:
            rec = self._record(slot)
            want = (rec.length + n_new + PAGE - 1) // PAGE
            for gi in range(len(self.groups)):
                need[gi] += max(0, want - len(rec.pages[gi]))
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.available:
                raise CacheFull(f"the step needs {need[gi]} more cache pages of {PAGE} tokens but only "
                                f"{g.pool.available} of {g.pool.capacity} are free (cache sized for "
                                f"{self.max_tokens} tokens)")
        for slot, n_new in plan:
            self.reserve(slot, n_new)

    def commit(self, slot: int, n_new: int) -> None:
        """The step has written ``n_new`` tokens of ``slot``: advance its length, and let window
        groups give back pages that no later query can see."""
        rec = self._record(slot)
        rec.length += n_new
        for gi, g in enumerate(self.groups):
            if rec.length > len(rec.pages[gi]) * PAGE:
                raise CacheError(f"slot {slot} was advanced to {rec.length} tokens beyond its reserved pages")
            first_needed = CACHE_KINDS[g.need.kind](g.need, rec.length)
            if first_needed >= PAGE:
                dead = first_needed // PAGE
                gone = [p for p in rec.pages[gi][:dead] if p >= 0]
                if gone:
                    g.pool.give_back(gone)
                    for i in range(dead):
                        rec.pages[gi][i] = -1

    def close(self, slot: int) -> None:
        rec = self._record(slot)
        for gi, g in enumerate(self.groups):
            g.pool.give_back([p for p in rec.pages[gi] if p >= 0])
        del self.records[slot]
        self.epoch += 1
        self.slots.give_back([slot])

    def close_all(self) -> None:
        for slot in list(self.records):
            self.close(slot)

    # ------------------------------------------------------------------ views for the step
    def pages(self, slot: int, group: int) -> List[int]:
        return self._record(slot).pages[group]

    def entry_storage(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """(K pool, V pool, group index) of a cache entry: pools are [pages, kv_heads, PAGE, head_dim]."""
        gi = self.group_of_entry[entry]
        g = self.groups[gi]
        i = g.index_of[entry]
        return g.k[i], g.v[i], gi

    def entry_state(self, entry: int) -> Optional[torch.Tensor]:
        """[slots, numel] float32 view of a cache entry's per-sequence state, or None."""
        if entry not in self.state_offsets:
            return None
        off, n = self.state_offsets[entry]
        return self.state[:, off:off + n]

    # ------------------------------------------------------------------ accounting
    def live_tokens(self) -> int:
        return sum(r.length for r in self.records.values())

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + self.state.numel() * 4

    def check(self) -> None:
        """Invariants: every page of every group is free or held by exactly one open sequence."""
        self.slots.check()
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = [p for r in self.records.values() for p in r.pages[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"a page of group {gi} is held by two sequences")
            if len(held) != g.pool.in_use:
                raise CacheError(f"group {gi}: {g.pool.in_use} pages are out but sequences hold {len(held)}")
        if set(self.records) != {i for i in range(self.max_slots) if self.slots._held[i]}:
            raise CacheError("open records and held slots differ")
