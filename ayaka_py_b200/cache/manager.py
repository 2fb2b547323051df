"""Pages, block tables and state slots.

Every KV group has a pool of pages of ``page_size`` tokens and, per request, a
row of a block table (logical page -> physical page).  Page 0 of each pool is a
permanent padding page: table entries that hold nothing point at it, and it is
never handed out (the reference keeps such a page too,
``memory/manager.py:140-142``).  A request holds a slot from ``open`` to
``close``; the slot indexes the block tables and the regions of fixed-size
state.  Pages come back when a request closes or is preempted, when a refused
step is rolled back, and, in a group with a window, when the window has passed
them.

A step is reserved as a whole (``reserve``: all entries or none, as the
reference rolls back a whole step, ``kvcache/manager.py:458-467``), run, then
committed.  The host tables are the truth; the step function copies the rows it
needs to the device.  All bookkeeping is host code and runs without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .spec import CacheGroupSpec


class OutOfPages(RuntimeError):
    """A step needs more pages than a group has free.  Nothing was changed."""

    def __init__(self, group: str, needed: int, free: int):
        super().__init__(f"cache group {group!r} needs {needed} pages, {free} are free")
        self.group, self.needed, self.free = group, needed, free


class NoFreeSlot(RuntimeError):
    """All request slots are taken."""


@dataclass
class Reservation:
    """A reserved step: its entries and the pages it took (for a rollback)."""
    entries: list[tuple[int, int, int]]                 # (slot, start, count)
    taken: list[list[tuple[int, int, int]]] = field(default_factory=list)  # per group: (slot, logical, page)
    settled: bool = False


class _PagePool:
    """Free pages of one group.  Last freed, first used: a page that came back
    is the next one handed out."""

    def __init__(self, pages: int):
        self.pages = pages
        self.free = list(range(pages - 1, 0, -1))        # page 0 is the padding page
        self.owner = np.full(pages, -1, dtype=np.int64)  # slot that holds the page, -1 free
        self.owner[0] = -2
        self.used_before = np.zeros(pages, dtype=bool)
        self.reused = 0
        self.high_water = 0

    def take(self, slot: int) -> int:
        page = self.free.pop()
        if self.owner[page] != -1:
            raise AssertionError(f"page {page} handed out while held by slot {self.owner[page]}")
        self.owner[page] = slot
        if self.used_before[page]:
            self.reused += 1
        self.used_before[page] = True
        self.high_water = max(self.high_water, self.pages - 1 - len(self.free))
        return page

    def give(self, page: int, slot: int) -> None:
        if page <= 0 or page >= self.pages:
            raise AssertionError(f"page {page} is not a page of this pool")
        if self.owner[page] != slot:
            raise AssertionError(f"page {page} freed by slot {slot}, held by {self.owner[page]}")
        self.owner[page] = -1
        self.free.append(page)


def pages_for_budget(groups: list[CacheGroupSpec], budget_bytes: int, *, page_size: int, max_requests: int,
                     max_len: int, step_tokens: int, dtype: torch.dtype) -> list[int]:
    """Pages per group (the padding page included; 0 for state groups) out of one byte
    budget.  A group whose layers read a window never holds more than the window plus
    one step's tokens per request, so it gets at most that; what remains is shared by
    the groups that keep every key so that each holds the same number of tokens (a
    request needs its tokens in all of them at once)."""
    item = torch.empty((), dtype=dtype).element_size()
    cost = [g.layers * page_size * g.need.elements_per_token() * item if isinstance(g.need, KVNeed) else 0
            for g in groups]
    pages = [0] * len(groups)
    left = int(budget_bytes)
    full = [i for i, g in enumerate(groups) if isinstance(g.need, KVNeed) and g.need.window is None]
    windowed = [i for i, g in enumerate(groups) if isinstance(g.need, KVNeed) and g.need.window is not None]
    per_token_page = sum(cost[i] for i in full + windowed)
    if not per_token_page:
        return pages
    even = left // per_token_page                       # pages each group would get if all were alike
    for i in windowed:
        per_request = -(-(min(max_len, groups[i].need.window + step_tokens)) // page_size) + 1
        pages[i] = max(2, min(even, max_requests * per_request + 1))
        left -= pages[i] * cost[i]
    if full:
        share = left // sum(cost[i] for i in full)
        for i in full:
            pages[i] = max(0, share)
    short = [groups[i].name for i in full + windowed if pages[i] < 2]
    if short:
        raise ValueError(f"a budget of {budget_bytes} bytes leaves no page for cache group(s) {short} "
                         f"(a page of each costs {[cost[i] for i in full + windowed]} bytes)")
    return pages


class CacheManager:
    def __init__(self, groups: list[CacheGroupSpec], *, kv_pages, page_size: int,
                 max_requests: int, max_len: int, dtype: torch.dtype = torch.float32,
                 device=None):
        """``kv_pages``: pages of every KV group (one number), or one number per group
        (see ``pages_for_budget``); the padding page counts.  ``device`` None: bookkeeping
        only (no tensors), for host tests."""
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError("page_size must be a power of two")
        self.groups = list(groups)
        self.page_size = page_size
        if isinstance(kv_pages, int):
            per_group = [kv_pages if isinstance(g.need, KVNeed) else 0 for g in self.groups]
        else:
            per_group = [int(n) for n in kv_pages]
            if len(per_group) != len(self.groups):
                raise ValueError(f"{len(per_group)} page counts for {len(self.groups)} cache groups")
        self.pages_of = per_group                       # pages of each group (0: a state group)
        self.kv_pages = min((n for n, g in zip(per_group, self.groups) if isinstance(g.need, KVNeed)), default=0)
        self.max_requests = max_requests
        self.max_len = max_len
        self.columns = -(-max_len // page_size)
        self.dtype, self.device = dtype, device

        self.free_slots = list(range(max_requests - 1, -1, -1))
        self.slot_of: dict[object, int] = {}
        self.request_of: dict[int, object] = {}
        self.length = np.zeros(max_requests, dtype=np.int64)      # committed tokens
        self.in_step = np.zeros(max_requests, dtype=bool)

        self.pools: list[_PagePool | None] = []
        self.tables: list[np.ndarray | None] = []
        self.first_page: list[np.ndarray | None] = []   # first logical page still held (window groups)
        self.num_pages: list[np.ndarray | None] = []    # logical pages ever assigned (= next logical index)
        self.kv: list[torch.Tensor | None] = []
        self.state: list[torch.Tensor | None] = []
        for g, n_pages in zip(self.groups, per_group):
            if isinstance(g.need, KVNeed):
                if n_pages < 2:
                    raise ValueError(f"cache group {g.name!r} needs at least 2 pages (one is the padding page)")
                self.pools.append(_PagePool(n_pages))
                self.tables.append(np.zeros((max_requests, self.columns), dtype=np.int32))
                self.first_page.append(np.zeros(max_requests, dtype=np.int64))
                self.num_pages.append(np.zeros(max_requests, dtype=np.int64))
                self.state.append(None)
                if device is not None:
                    # keys [layer, page, token in page, kv head, head dim]; values the same with their own heads and size
                    self.kv.append((
                        torch.zeros((g.layers, n_pages, page_size, g.need.kv_heads, g.need.head_dim), dtype=dtype, device=device),
                        torch.zeros((g.layers, n_pages, page_size, g.need.v_heads, g.need.v_dim), dtype=dtype, device=device)))
                else:
                    self.kv.append(None)
            elif isinstance(g.need, StateNeed):
                self.pools.append(None)
                self.tables.append(None)
                self.first_page.append(None)
                self.num_pages.append(None)
                self.kv.append(None)
                # one spare slot at index max_requests: where padding lanes of a graph step write
                self.state.append(None if device is None else torch.zeros(
                    (g.layers, max_requests + 1, *g.need.shape), dtype=g.need.dtype, device=device))
            else:
                raise TypeError(f"group {g.name}: unknown need {g.need!r}")

    # ------------------------------------------------------------- requests --
    def open(self, request_id) -> int:
        if request_id in self.slot_of:
            raise KeyError(f"request {request_id!r} is already open")
        if not self.free_slots:
            raise NoFreeSlot(f"all {self.max_requests} request slots are taken")
        slot = self.free_slots.pop()
        self.slot_of[request_id] = slot
        self.request_of[slot] = request_id
        self.length[slot] = 0
        for state in self.state:
            if state is not None:
                state[:, slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """Gives back every page and the slot."""
        self._check_slot(slot)
        if self.in_step[slot]:
            raise RuntimeError(f"slot {slot} is inside a reserved step")
        self._drop_pages(slot)
        request_id = self.request_of.pop(slot)
        del self.slot_of[request_id]
        self.length[slot] = 0
        self.free_slots.append(slot)

    def preempt(self, slot: int) -> None:
        """Gives back every page but keeps the slot; the request starts again
        at token 0 (recompute preemption, ``memory/manager.py:1283-1370``)."""
        self._check_slot(slot)
        if self.in_step[slot]:
            raise RuntimeError(f"slot {slot} is inside a reserved step")
        self._drop_pages(slot)
        self.length[slot] = 0
        for state in self.state:
            if state is not None:
                state[:, slot].zero_()

    def _drop_pages(self, slot: int) -> None:
        for g, pool in enumerate(self.pools):
            if pool is None:
                continue
            for logical in range(int(self.first_page[g][slot]), int(self.num_pages[g][slot])):
                pool.give(int(self.tables[g][slot, logical]), slot)
            self.tables[g][slot, :] = 0
            self.first_page[g][slot] = 0
            self.num_pages[g][slot] = 0

    def _check_slot(self, slot: int) -> None:
        if slot not in self.request_of:
            raise KeyError(f"slot {slot} is not open")

    # ---------------------------------------------------------------- steps --
    def pages_needed(self, entries) -> list[int]:
        """New pages per group that ``entries`` would take (0 for state groups)."""
        out = []
        for g, pool in enumerate(self.pools):
            if pool is None:
                out.append(0)
                continue
            need = 0
            for slot, start, count in entries:
                need += self._first_and_new(g, slot, start, count)[1]
            out.append(need)
        return out

    def _first_and_new(self, g: int, slot: int, start: int, count: int) -> tuple[int, int]:
        end_pages = -(-(start + count) // self.page_size)
        have = int(self.num_pages[g][slot])
        return have, max(0, end_pages - have)

    def free_pages(self, g: int = 0) -> int:
        pool = self.pools[g]
        return 0 if pool is None else len(pool.free)

    def pages_held(self, slots) -> list:
        """Per group: the pages that each of ``slots`` holds, as an array (None for a group of
        state slots).  With ``free_pages`` this lets a planner try portions of other sizes by
        arithmetic and call ``reserve`` once, for the one that fits."""
        slots_a = np.fromiter((int(s) for s in slots), dtype=np.int64, count=len(slots))
        return [None if pool is None else self.num_pages[g][slots_a].astype(np.int64) for g, pool in enumerate(self.pools)]

    def reserve(self, entries) -> Reservation:
        """entries: (slot, start, count).  Each must start at the request's
        committed length.  All or nothing: raises ``OutOfPages`` with nothing
        changed when any group lacks pages."""
        entries = [(int(s), int(a), int(c)) for s, a, c in entries]
        seen = set()
        for slot, start, count in entries:
            self._check_slot(slot)
            if slot in seen:
                raise ValueError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if self.in_step[slot]:
                raise RuntimeError(f"slot {slot} is already inside a reserved step")
            if count < 1:
                raise ValueError("an entry must bring at least one token")
            if start != self.length[slot]:
                raise ValueError(f"slot {slot}: entry starts at {start}, the cache holds {self.length[slot]} tokens")
            if start + count > self.max_len:
                raise ValueError(f"slot {slot}: {start + count} tokens exceed the limit of {self.max_len}")
        # pages that each entry's last token needs, against the pages its request has (all entries at once)
        slots_a = np.fromiter((e[0] for e in entries), dtype=np.int64, count=len(entries))
        end_pages = -(-np.fromiter((e[1] + e[2] for e in entries), dtype=np.int64, count=len(entries)) // self.page_size)
        news = []
        for g, pool in enumerate(self.pools):
            if pool is None:
                news.append(None)
                continue
            new = np.maximum(0, end_pages - self.num_pages[g][slots_a])
            need = int(new.sum())
            if need > len(pool.free):
                raise OutOfPages(self.groups[g].name, need, len(pool.free))
            news.append(new)
        res = Reservation(entries)
        for g, pool in enumerate(self.pools):
            taken = []
            if pool is not None:
                for i in np.flatnonzero(news[g]):          # most decode entries need no new page
                    slot = int(slots_a[i])
                    have = int(self.num_pages[g][slot])
                    for logical in range(have, have + int(news[g][i])):
                        page = pool.take(slot)
                        self.tables[g][slot, logical] = page
                        taken.append((slot, logical, page))
                    self.num_pages[g][slot] = have + int(news[g][i])
            res.taken.append(taken)
        self.in_step[slots_a] = True
        return res

    def commit(self, res: Reservation) -> None:
        """The step ran: lengths advance; pages that a window has passed return."""
        self._settle(res)
        if res.entries:
            slots_a = np.fromiter((e[0] for e in res.entries), dtype=np.int64, count=len(res.entries))
            self.length[slots_a] = np.fromiter((e[1] + e[2] for e in res.entries), dtype=np.int64, count=len(res.entries))
        for g, group in enumerate(self.groups):
            if self.pools[g] is None or group.need.window is None:
                continue
            for slot, start, count in res.entries:
                # The next query sits at position L and reads keys > L - window.
                first_needed = max(0, int(self.length[slot]) - group.need.window + 1) // self.page_size
                for logical in range(int(self.first_page[g][slot]), min(first_needed, int(self.num_pages[g][slot]))):
                    self.pools[g].give(int(self.tables[g][slot, logical]), slot)
                    self.tables[g][slot, logical] = 0
                self.first_page[g][slot] = max(int(self.first_page[g][slot]),
                                               min(first_needed, int(self.num_pages[g][slot])))

    def rollback(self, res: Reservation) -> None:
        """The step did not run: the pages it took return, lengths stay."""
        self._settle(res)
        for g, taken in enumerate(res.taken):
            for slot, logical, page in reversed(taken):
                self.pools[g].give(page, slot)
                self.tables[g][slot, logical] = 0
                self.num_pages[g][slot] = min(int(self.num_pages[g][slot]), logical)

    def _settle(self, res: Reservation) -> None:
        if res.settled:
            raise RuntimeError("this step was already committed or rolled back")
        res.settled = True
        if res.entries:
            self.in_step[[e[0] for e in res.entries]] = False

    # ---------------------------------------------------------------- views --
    def table_rows(self, g: int, slots) -> np.ndarray:
        """Block-table rows [len(slots), columns] int32 of a KV group."""
        return self.tables[g][np.asarray(slots, dtype=np.int64)]

    def kv_layer(self, g: int, layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(K, V) pages of one layer: [pages, page_size, kv_heads, head_dim] and the same with the
        values' heads and size."""
        keys, values = self.kv[g]
        return keys[layer], values[layer]

    def state_layer(self, g: int, layer: int) -> torch.Tensor:
        """State of one layer: [max_requests + 1, *shape], indexed by slot (the last is a spare)."""
        return self.state[g][layer]

    def bytes_per_token(self) -> int:
        total = 0
        item = torch.empty((), dtype=self.dtype).element_size()
        for g in self.groups:
            if isinstance(g.need, KVNeed):
                total += g.layers * g.need.elements_per_token() * item
        return total

    # ---------------------------------------------------------- diagnostics --
    def stats(self) -> dict:
        out = {"open_requests": len(self.slot_of), "free_slots": len(self.free_slots), "groups": {}}
        for g, pool in enumerate(self.pools):
            if pool is not None:
                out["groups"][self.groups[g].name] = {
                    "pages": pool.pages - 1, "free": len(pool.free),
                    "high_water": pool.high_water, "reused": pool.reused}
        return out

    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held; tables agree with owners."""
        if len(set(self.free_slots)) != len(self.free_slots):
            raise AssertionError("a slot is free twice")
        if set(self.free_slots) & set(self.request_of):
            raise AssertionError("a slot is both free and open")
        if len(self.free_slots) + len(self.request_of) != self.max_requests:
            raise AssertionError("a slot is lost")
        for g, pool in enumerate(self.pools):
            if pool is None:
                continue
            free = pool.free
            if len(set(free)) != len(free):
                raise AssertionError(f"group {g}: a page is free twice")
            held = {}
            for slot in self.request_of:
                for logical in range(int(self.first_page[g][slot]), int(self.num_pages[g][slot])):
                    page = int(self.tables[g][slot, logical])
                    if page <= 0:
                        raise AssertionError(f"group {g}: slot {slot} logical page {logical} holds no page")
                    if page in held:
                        raise AssertionError(f"group {g}: page {page} held by slots {held[page]} and {slot}")
                    held[page] = slot
                    if pool.owner[page] != slot:
                        raise AssertionError(f"group {g}: page {page} owner {pool.owner[page]} != slot {slot}")
            if set(free) & set(held):
                raise AssertionError(f"group {g}: a page is both free and held")
            if len(free) + len(held) != pool.pages - 1:
                raise AssertionError(
                    f"group {g}: {pool.pages - 1 - len(free) - len(held)} pages lost")
            for slot in range(self.max_requests):
                if slot not in self.request_of and self.tables[g][slot].any():
                    raise AssertionError(f"group {g}: closed slot {slot} still has table entries")

    def assert_clean(self) -> None:
        """Every page and slot is free (after all requests ended)."""
        self.check_invariants()
        if self.request_of:
            raise AssertionError(f"requests still open: {sorted(map(str, self.request_of.values()))}")
        for g, pool in enumerate(self.pools):
            if pool is not None and len(pool.free) != pool.pages - 1:
                raise AssertionError(f"group {g}: {pool.pages - 1 - len(pool.free)} pages not returned")
