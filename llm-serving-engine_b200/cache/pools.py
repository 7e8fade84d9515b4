"""Device tensors of the cache and the grouping of cache layers by what they keep.

Keys and values of a group live in one tensor ``[layers, 2, pages, kv_heads, page_tokens,
head_dim]``: the rows of one (page, head) are contiguous (``page_tokens * head_dim`` elements), so
a kernel that walks a request's context for one head reads whole contiguous runs. Fixed-size
per-request state lives in ``[layers, max_requests, *shape]`` tensors, indexed by state slot.

Every key/value tensor has one page more than the manager hands out, and every state tensor one
slot more (``spare_page(group)``, ``spare_slot``): rows that only pad a captured batch to its fixed
size write there, where no request ever reads.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import PagedKVNeed, StateNeed
from .manager import KVGroupSpec, StateGroupSpec


def group_cache_layers(needs: dict[int, object], page_tokens: int):
    """Sort cache layers into key/value groups (same heads, head size, window and page dtype) and
    state groups."""
    kv: dict[tuple, list[int]] = {}
    st: dict[tuple, list[int]] = {}
    for cid in sorted(needs):
        need = needs[cid]
        if need is None:
            continue
        if isinstance(need, PagedKVNeed):
            kv.setdefault((need.num_kv_heads, need.head_dim, need.window, need.dtype), []).append(cid)
        elif isinstance(need, StateNeed):
            st.setdefault((tuple(need.shape), need.dtype), []).append(cid)
        else:
            raise TypeError(f"cache layer {cid}: unknown need {need!r}")
    kv_groups = [
        KVGroupSpec(tuple(ids), nk, d, w, page_tokens, dt) for (nk, d, w, dt), ids in kv.items()
    ]
    state_groups = [StateGroupSpec(tuple(ids), shape, dt) for (shape, dt), ids in st.items()]
    return kv_groups, state_groups


def pages_for_memory(groups, mem_bytes: int, dtype_bytes: int, max_len: int, max_portion: int):
    """Split ``mem_bytes`` between the groups in proportion to what one full-length request holds."""
    weights = [g.bytes_per_token(dtype_bytes) * g.live_tokens(max_len, max_portion) for g in groups]
    total = sum(weights) or 1
    out = []
    for g, w in zip(groups, weights):
        page_bytes = g.bytes_per_token(dtype_bytes) * g.page_tokens
        out.append(max(1, int(mem_bytes * w / total) // page_bytes))
    return out


@dataclass
class CacheView:
    """What one run of a layer sees of the cache."""

    group: int  # index of the key/value group (selects the block table), -1 if none
    page_tokens: int
    k: torch.Tensor | None  # [pages, kv_heads, page_tokens, head_dim]
    v: torch.Tensor | None
    state: torch.Tensor | None  # [max_requests, *shape]
    writes: bool


class CachePools:
    def __init__(self, kv_groups, state_groups, num_pages, max_requests, dtype, device) -> None:
        self.kv_groups = list(kv_groups)
        self.state_groups = list(state_groups)
        self.num_pages = list(num_pages)
        self.max_requests = max_requests
        self.kv = [
            torch.zeros(
                len(g.cache_ids), 2, n + 1, g.num_kv_heads, g.page_tokens, g.head_dim,
                dtype=g.dtype or dtype, device=device,
            )
            for g, n in zip(self.kv_groups, self.num_pages)
        ]
        self.state = [
            torch.zeros(len(g.cache_ids), max_requests + 1, *g.shape, dtype=g.dtype, device=device)
            for g in self.state_groups
        ]
        self._where: dict[int, tuple[str, int, int]] = {}
        for gi, g in enumerate(self.kv_groups):
            for li, cid in enumerate(g.cache_ids):
                self._where[cid] = ("kv", gi, li)
        for gi, g in enumerate(self.state_groups):
            for li, cid in enumerate(g.cache_ids):
                self._where[cid] = ("state", gi, li)

    def view(self, cache_id: int, writes: bool) -> CacheView:
        where = self._where.get(cache_id)
        if where is None:
            return CacheView(-1, 0, None, None, None, writes)
        kind, gi, li = where
        if kind == "kv":
            t = self.kv[gi][li]
            return CacheView(gi, self.kv_groups[gi].page_tokens, t[0], t[1], None, writes)
        return CacheView(-1, 0, None, None, self.state[gi][li], writes)

    def spare_page(self, group: int) -> int:
        """A page of ``group`` that the manager never hands out."""
        return self.num_pages[group]

    @property
    def spare_slot(self) -> int:
        """A state slot that no request ever holds."""
        return self.max_requests

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + self.state)
