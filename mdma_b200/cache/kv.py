"""The cache: a slot per live sequence, keys and values per cache site in pages.

A *site* is one run of a layer in the model's schedule that keeps keys and
values.  Sites with the same need (heads, head size, window) form a *group*
with storage of its own: a pool of pages `[sites, pages, page_size, kv_heads,
head_dim]` for keys and one for values, a free list of pages and one page
table `[slots, max_pages]`.  A sequence holds a slot, and in every group the
pages that cover its length; groups with a window give pages back once every
key in them has left the window.  Slots and pages go back to the free lists
when a sequence ends and are handed out again.  Next to the pages lies
fixed-size per-sequence state `[slots, ...]` for sites that declare some; it
is zeroed when a slot is taken.

The reference keeps one cache object per sequence with per-layer widths,
windows and optional fixed-size state (src/kv_cache.rs:16-131, 279-292); this
is the same inventory for many sequences at once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .slots import CacheFull, FreeList


@dataclass(frozen=True)
class KVNeed:
    """What a mixer asks of the cache for one site."""
    n_kv_heads: int
    head_dim: int
    window: int = 0          # 0: every key is kept; n: only the last n keys are read


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence for one site."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class KVView:
    """What a mixer gets for its site: this site's pages and how to index them."""
    k: Optional[torch.Tensor]            # [pages, page_size, kv_heads, head_dim]
    v: Optional[torch.Tensor]
    page_table: Optional[torch.Tensor]   # int32 [slots, max_pages], on the device
    page_size: int
    max_pages: int
    window: int
    state: Optional[torch.Tensor] = None  # [slots, *shape]


class CacheGroup:
    def __init__(self, need: KVNeed, sites: list[int], n_pages: int, n_slots: int, max_pages: int,
                 page_size: int, dtype: torch.dtype, alloc):
        self.need, self.sites = need, sites
        self.n_pages, self.page_size, self.max_pages = n_pages, page_size, max_pages
        self.pages = FreeList(n_pages, "cache page")
        self.table_host = np.zeros((n_slots, max_pages), dtype=np.int32)
        self.seq_pages: dict[int, dict[int, int]] = {}      # slot -> {page index in sequence: page}
        self.dirty: set[int] = set()
        shape = (len(sites), n_pages, page_size, need.n_kv_heads, need.head_dim)
        self.bytes = 2 * int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        # `alloc(shape, dtype)` hands out zeroed device memory, or None when only sizes are wanted
        self.k = alloc(shape, dtype)
        self.v = alloc(shape, dtype)
        self.table_dev = alloc((n_slots, max_pages), torch.int32)

    def grow(self, slot: int, old_len: int, new_len: int) -> None:
        """Make sure pages cover positions [.., new_len) of `slot` for this step."""
        have = self.seq_pages.setdefault(slot, {})
        if new_len <= 0:
            return
        first_needed = 0
        if self.need.window:
            # the earliest key any token of this step reads
            first_needed = max(0, old_len + 1 - self.need.window) // self.page_size
        last = (new_len - 1) // self.page_size
        if last >= self.max_pages:
            raise CacheFull(f"a sequence of {new_len} tokens needs more than {self.max_pages} pages")
        # the pages that cover [first_needed, old_len) are held already: look from the last of them on
        start = max(first_needed, (old_len - 1) // self.page_size) if old_len > 0 else first_needed
        missing = [p for p in range(start, last + 1) if p not in have]
        fresh = self.pages.acquire_many(len(missing))
        for p, page in zip(missing, fresh):
            have[p] = page
            self.table_host[slot, p] = page
        if missing:
            self.dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Give back pages whose keys have all left the window of every later token."""
        if not self.need.window:
            return
        have = self.seq_pages.get(slot, {})
        first_live = max(0, length + 1 - self.need.window) // self.page_size
        for p in [p for p in have if p < first_live]:
            self.pages.release(have.pop(p))

    def release(self, slot: int) -> None:
        for page in self.seq_pages.pop(slot, {}).values():
            self.pages.release(page)
        self.dirty.discard(slot)

    def sync_tables(self) -> None:
        """Copy the page-table rows that changed to the device."""
        if self.table_dev is None or not self.dirty:
            return
        for row in sorted(self.dirty):      # straight into the table: no device memory is taken for the copy
            self.table_dev[row].copy_(torch.from_numpy(self.table_host[row]))
        self.dirty.clear()


class SequenceCache:
    """Slots, page groups and per-sequence state for one engine."""

    def __init__(self, kv_needs: list[Optional[KVNeed]], state_needs: list[Optional[StateNeed]],
                 max_tokens: int, max_slots: int, max_context: int, dtype: torch.dtype, device,
                 page_size: int = 64, allocate: bool = True, alloc=None):
        """`alloc(shape, dtype)`: where pools, tables and state come from (an engine passes its arena;
        it may return None to add up sizes only).  Without it they are allocated here, or, with
        `allocate=False`, not at all."""
        assert len(kv_needs) == len(state_needs)
        if alloc is None:
            alloc = ((lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)) if allocate
                     else (lambda shape, dt: None))
        if page_size <= 0 or max_tokens <= 0 or max_slots <= 0 or max_context <= 0:
            raise ValueError("cache sizes must be positive")
        self.page_size, self.max_context, self.max_slots = page_size, max_context, max_slots
        self.dtype, self.device = dtype, device
        self.n_pages = -(-max_tokens // page_size)
        self.max_pages = -(-max_context // page_size)
        self.slots = FreeList(max_slots, "sequence slot")
        self.lengths: dict[int, int] = {}
        self.groups: list[CacheGroup] = []
        self.site_group: dict[int, tuple[int, int]] = {}
        by_need: dict[KVNeed, list[int]] = {}
        for site, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(site)
        for need, sites in by_need.items():
            g = CacheGroup(need, sites, self.n_pages, max_slots, self.max_pages, page_size, dtype, alloc)
            for j, site in enumerate(sites):
                self.site_group[site] = (len(self.groups), j)
            self.groups.append(g)
        self.states: dict[int, torch.Tensor] = {}
        self.state_bytes = 0
        for site, need in enumerate(state_needs):
            if need is None:
                continue
            n = int(np.prod(need.shape)) * max_slots * torch.empty((), dtype=need.dtype).element_size()
            self.state_bytes += n
            state = alloc((max_slots, *need.shape), need.dtype)
            if state is not None:
                self.states[site] = state

    # ---- sizes ---------------------------------------------------------
    @property
    def bytes(self) -> int:
        tables = sum(g.table_host.nbytes for g in self.groups)
        return sum(g.bytes for g in self.groups) + self.state_bytes + tables

    # ---- sequences -----------------------------------------------------
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.lengths[slot] = 0
        for state in self.states.values():
            state[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)
        for g in self.groups:
            g.release(slot)
        del self.lengths[slot]

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    def can_extend(self, extensions: dict[int, int]) -> Optional[str]:
        """None if every slot in {slot: new tokens} can grow, else the reason."""
        for g in self.groups:
            want = 0
            for slot, n_new in extensions.items():
                old = self.lengths[slot]
                if old + n_new > self.max_context:
                    return (f"sequence in slot {slot} would reach {old + n_new} tokens, "
                            f"beyond the context of {self.max_context}")
                have = g.seq_pages.get(slot, {})
                first = max(0, old + 1 - g.need.window) // self.page_size if g.need.window else 0
                if old > 0:                    # pages up to the one that holds position old - 1 are held
                    first = max(first, (old - 1) // self.page_size)
                last = (old + n_new - 1) // self.page_size
                want += sum(1 for p in range(first, last + 1) if p not in have)
            if want > g.pages.free_count:
                return (f"the step needs {want} more cache pages of {self.page_size} tokens, "
                        f"{g.pages.free_count} of {g.n_pages} are free")
        return None

    def extend(self, extensions: dict[int, int]) -> None:
        """Reserve pages so that each slot can take its new tokens; all or nothing."""
        why = self.can_extend(extensions)
        if why:
            raise CacheFull(why)
        for slot, n_new in extensions.items():
            old = self.lengths[slot]
            for g in self.groups:
                g.grow(slot, old, old + n_new)
        for g in self.groups:
            g.sync_tables()

    def commit(self, extensions: dict[int, int]) -> None:
        """The step ran: the new tokens are part of the sequences."""
        for slot, n_new in extensions.items():
            self.lengths[slot] += n_new
            for g in self.groups:
                g.trim(slot, self.lengths[slot])

    def truncate(self, slot: int, length: int) -> None:
        """Forget the tokens of `slot` from position `length` on (pages beyond go back to the free
        list).  Refused when the cache holds fixed-size state or a windowed group has already given
        pages of the kept part back: neither can be rewound (the reference's rule for its `rewind`,
        src/kv_cache.rs:255-276)."""
        old = self.lengths[slot]
        if not 0 <= length <= old:
            raise ValueError(f"cannot truncate a sequence of {old} tokens to {length}")
        if self.states:
            raise ValueError("a cache with fixed-size per-sequence state cannot be rewound")
        for g in self.groups:
            have = g.seq_pages.get(slot, {})
            if g.need.window:
                first_needed = max(0, length + 1 - g.need.window) // self.page_size
                last = (length - 1) // self.page_size if length else -1
                if any(p not in have for p in range(first_needed, last + 1)):
                    raise ValueError("a windowed group has already released pages of the kept part")
            keep_last = (length - 1) // self.page_size if length else -1
            for p in [p for p in have if p > keep_last]:
                g.pages.release(have.pop(p))
        self.lengths[slot] = length

    def view(self, site: int, state_site: Optional[int] = None) -> KVView:
        """Pages of `site`; the fixed-size state of `state_site` (default: the same site)."""
        state = self.states.get(site if state_site is None else state_site)
        if site not in self.site_group:
            return KVView(None, None, None, self.page_size, self.max_pages, 0, state)
        gi, j = self.site_group[site]
        g = self.groups[gi]
        return KVView(g.k[j] if g.k is not None else None, g.v[j] if g.v is not None else None,
                      g.table_dev, self.page_size, self.max_pages, g.need.window, state)

    def poison_unused(self, value: float = float("nan")) -> None:
        """Testing aid: overwrite every cache row that no live sequence owns (all rows of free
        pages, and the rows at and beyond each sequence's length in the pages it holds) with
        `value`.  Results must not change: a kernel may fetch such rows with a tile but must not
        let them reach its output (the reference's rule is `written` against `len`,
        src/kv_cache.rs:246-268)."""
        for g in self.groups:
            if g.k is None:
                continue
            free = sorted(set(range(g.n_pages)) - set(g.pages.held))
            if free:
                idx = torch.as_tensor(free, dtype=torch.long, device=g.k.device)
                g.k.index_fill_(1, idx, value)
                g.v.index_fill_(1, idx, value)
            for slot, have in g.seq_pages.items():
                length = self.lengths.get(slot, 0)
                for p, page in have.items():
                    first = max(0, length - p * self.page_size)
                    if first < self.page_size:
                        g.k[:, page, first:] = value
                        g.v[:, page, first:] = value

    def check(self) -> None:
        """Invariants: no slot or page lost, held twice, or owned by two sequences."""
        self.slots.check()
        assert set(self.lengths) == set(self.slots.held)
        for g in self.groups:
            g.pages.check()
            owned = [page for pages in g.seq_pages.values() for page in pages.values()]
            assert len(owned) == len(set(owned)), "a page belongs to two sequences"
            assert set(owned) == set(g.pages.held), "held pages and owned pages differ"
            assert set(g.seq_pages) <= set(self.slots.held), "pages owned by a slot that is free"
