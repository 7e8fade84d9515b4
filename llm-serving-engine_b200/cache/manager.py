"""Cache manager: which pages and which state slot each live request holds.

Host-side bookkeeping only (integers, no tensors); the tensors live in
:class:`llmserve_b200.cache.pools.CachePools`.

* Cache layers with the same need form a *group* (:class:`KVGroupSpec`). Each group has its own
  page pool and each request has one block table per group: entry ``i`` is the page that holds the
  request's tokens ``i*page_tokens .. (i+1)*page_tokens-1`` for every layer of the group.
* A group with a window gives a page back as soon as no later query can read it: after ``c``
  tokens are computed, the next query sits at position ``c`` and reads keys ``>= c-window+1``, so
  page ``i`` is released once ``(i+1)*page_tokens <= c-window+1``. Its table entry becomes -1.
* Each live request also holds one *state slot*, an index below ``max_requests``, which selects
  its row in every fixed-size per-request state tensor. The Llama architecture keeps nothing
  there; the slot exists so that a mixer with a recurrent state finds a place for it.
* Everything a request holds is returned by :meth:`release` (finish, abort or preemption), pages
  in reverse table order to the tail of the free list (src/llmserve/block_manager.py:98-108).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .allocator import OutOfPages, PageAllocator

RELEASED = -1


@dataclass(frozen=True)
class KVGroupSpec:
    """Cache layers that keep keys and values with the same shape and the same window."""

    cache_ids: tuple[int, ...]
    num_kv_heads: int
    head_dim: int
    window: int  # 0: every token is kept
    page_tokens: int
    dtype: object = None  # of the pages; None: the model's compute dtype

    def bytes_per_token(self, dtype_bytes: int) -> int:
        """``dtype_bytes``: element size of the compute dtype (used unless the group names its own)."""
        if self.dtype is not None:
            dtype_bytes = self.dtype.itemsize
        return 2 * len(self.cache_ids) * self.num_kv_heads * self.head_dim * dtype_bytes

    def live_tokens(self, max_len: int, max_portion: int = 1) -> int:
        """Most tokens of one request that the group holds at a time (rounded up to pages).

        With a window, a step of ``max_portion`` tokens starting at position c needs keys
        ``c-window+1 .. c+max_portion-1``, which may straddle one more page at the front.
        """
        if self.window <= 0:
            n = max_len
        else:
            n = min(max_len, self.window - 1 + max_portion + self.page_tokens)
        return -(-n // self.page_tokens) * self.page_tokens


@dataclass(frozen=True)
class StateGroupSpec:
    """Cache layers that keep one fixed-size tensor per request."""

    cache_ids: tuple[int, ...]
    shape: tuple[int, ...]
    dtype: object


@dataclass
class _Held:
    slot: int
    computed: int = 0
    tables: list[list[int]] = field(default_factory=list)  # one per group
    epoch: int = 0  # number of the admission; a new holder of the same slot has another one
    # the same tables as int32 arrays with room to grow (what a step's batch is built from)
    arrays: list[np.ndarray] = field(default_factory=list)

    def append_pages(self, g: int, pages: list[int]) -> None:
        table = self.tables[g]
        n = len(table)
        table.extend(pages)
        arr = self.arrays[g]
        if len(table) > arr.shape[0]:
            room = np.empty(max(len(table), 2 * arr.shape[0]), np.int32)
            arr = self.arrays[g] = np.concatenate([arr, room])
        arr[n : len(table)] = pages


class CacheManager:
    def __init__(self, groups: list[KVGroupSpec], num_pages: list[int], max_requests: int) -> None:
        if len(groups) != len(num_pages):
            raise ValueError("one page count per group is needed")
        if max_requests < 1:
            raise ValueError("max_requests must be at least 1")
        self.groups = list(groups)
        self.pools = [PageAllocator(n) for n in num_pages]
        self.max_requests = max_requests
        self.free_slots: list[int] = list(range(max_requests - 1, -1, -1))
        self.held: dict[object, _Held] = {}
        self._epochs = 0

    # ------------------------------------------------------------------ admission
    def is_live(self, rid) -> bool:
        return rid in self.held

    def has_free_slot(self) -> bool:
        return bool(self.free_slots)

    def admit(self, rid) -> int:
        """Give ``rid`` a state slot and empty block tables. Returns the slot."""
        if rid in self.held:
            raise KeyError(f"request {rid!r} is already live")
        if not self.free_slots:
            raise OutOfPages("no free state slot")
        slot = self.free_slots.pop()
        self._epochs += 1
        self.held[rid] = _Held(slot, 0, [[] for _ in self.groups], self._epochs,
                               [np.empty(16, np.int32) for _ in self.groups])
        return slot

    # ------------------------------------------------------------------ capacity
    def _new_pages(self, h: _Held, g: int, n: int) -> int:
        spec = self.groups[g]
        need = -(-(h.computed + n) // spec.page_tokens)
        return max(0, need - len(h.tables[g]))

    def pages_needed(self, rid, n: int) -> list[int]:
        """Pages each group must still hand out before ``n`` more tokens of ``rid`` can run."""
        h = self.held.get(rid) or _Held(-1, 0, [[] for _ in self.groups])
        return [self._new_pages(h, g, n) for g in range(len(self.groups))]

    def can_allocate(self, rid, n: int) -> bool:
        if rid not in self.held and not self.free_slots:
            return False
        need = self.pages_needed(rid, n)
        return all(need[g] <= self.pools[g].num_free for g in range(len(self.groups)))

    def fits_at_all(self, total_tokens: int, max_portion: int = 1) -> bool:
        """Could one request of ``total_tokens`` ever run with every other page free?"""
        return all(
            -(-spec.live_tokens(total_tokens, max_portion) // spec.page_tokens) <= pool.num_pages
            for spec, pool in zip(self.groups, self.pools)
        )

    # ------------------------------------------------------------------ growth and release
    def allocate(self, rid, n: int) -> None:
        """Make room for tokens ``computed .. computed+n-1`` of ``rid`` in every group."""
        h = self.held[rid]
        need = [self._new_pages(h, g, n) for g in range(len(self.groups))]
        for g, k in enumerate(need):
            if k > self.pools[g].num_free:
                raise OutOfPages(
                    f"group {g}: request {rid!r} needs {k} pages, {self.pools[g].num_free} are free"
                )
        for g, k in enumerate(need):
            if k:
                h.append_pages(g, [self.pools[g].allocate() for _ in range(k)])

    def try_allocate(self, rid, n: int) -> bool:
        """:meth:`allocate` for a live request if every group has the pages; else take nothing."""
        h = self.held[rid]
        end = h.computed + n
        need = None
        for g, spec in enumerate(self.groups):
            k = -(-end // spec.page_tokens) - len(h.tables[g])
            if k > 0:
                if k > self.pools[g].num_free:
                    return False
                need = need or []
                need.append((g, k))
        if need:
            for g, k in need:
                h.append_pages(g, [self.pools[g].allocate() for _ in range(k)])
        return True

    def commit(self, rid, n: int) -> None:
        """``n`` more tokens of ``rid`` are in the cache; give back pages a window has passed."""
        h = self.held[rid]
        h.computed += n
        for g, spec in enumerate(self.groups):
            if spec.window <= 0:
                continue
            assert h.computed <= len(h.tables[g]) * spec.page_tokens, "committed past the table"
            first_needed = h.computed - spec.window + 1
            i = 0
            table = h.tables[g]
            while (i + 1) * spec.page_tokens <= first_needed and i < len(table):
                if table[i] != RELEASED:
                    self.pools[g].release(table[i])
                    table[i] = RELEASED
                    h.arrays[g][i] = RELEASED
                i += 1

    def release(self, rid) -> None:
        """Give back every page and the state slot of ``rid`` (finish, abort or preemption)."""
        h = self.held.pop(rid)
        for g, table in enumerate(h.tables):
            for p in reversed(table):
                if p != RELEASED:
                    self.pools[g].release(p)
        self.free_slots.append(h.slot)

    # ------------------------------------------------------------------ queries
    def block_table(self, rid, group: int = 0) -> list[int]:
        return self.held[rid].tables[group]

    def table_array(self, rid, group: int = 0) -> np.ndarray:
        """The block table as an int32 array (a view: valid until the table next grows)."""
        h = self.held[rid]
        return h.arrays[group][: len(h.tables[group])]

    def state_slot(self, rid) -> int:
        return self.held[rid].slot

    def epoch(self, rid) -> int:
        return self.held[rid].epoch

    def num_computed(self, rid) -> int:
        return self.held[rid].computed

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def num_pages(self, group: int = 0) -> int:
        return self.pools[group].num_pages

    def usage(self) -> float:
        total = sum(p.num_pages for p in self.pools)
        return 1.0 - sum(p.num_free for p in self.pools) / total

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; no slot lost or held twice."""
        for g, pool in enumerate(self.pools):
            pool.check_invariants()
            held = [p for h in self.held.values() for p in h.tables[g] if p != RELEASED]
            assert len(held) == len(set(held)), f"group {g}: a page is held twice"
            assert all(pool.ref[p] == 1 for p in held), f"group {g}: a held page is marked free"
            assert len(held) + pool.num_free == pool.num_pages, f"group {g}: a page is lost"
        slots = [h.slot for h in self.held.values()]
        assert len(slots) == len(set(slots)), "a state slot is held twice"
        assert sorted(slots + self.free_slots) == list(range(self.max_requests)), "a slot is lost"
        for rid, h in self.held.items():
            for g, spec in enumerate(self.groups):
                assert h.computed <= len(h.tables[g]) * spec.page_tokens, f"{rid!r}: table too short"
                assert h.arrays[g][: len(h.tables[g])].tolist() == h.tables[g], f"{rid!r}: array differs"
