"""The cache manager: keys and values in pages, a block table for each request, and slots
for per-request state of fixed size. Host-side bookkeeping only; the device tensors that the
page ids index live in `hipinfer_b200/cache/storage.py`.

Layers are put into GROUPS by what they need. A group of kind "full" keeps every key of a
request; a group of kind "window" keeps the last `window` keys, and its pages are given back
as soon as every position on them has fallen out of the window of all tokens still to come.
A kind is a RETENTION RULE, a function from (group, position of the next query) to the ranges of
positions that no later query can see; `register_retention` adds another. What a layer keeps
per token is a tuple of PLANES (name, heads, width): keys and values of one shape for attention,
any other set for a mixer that keeps a latent or keys and values of different widths.
Each group has a page pool of its own and each request one block table per group, indexed by
logical page (position // page_size); a released entry reads -1. All pages return to their
pool when the request ends. A freed page is handed out again, lowest id first, so that which
page a request gets is reproducible.

Beside the pages there are STATE SLOTS: one integer per live request, handed out at admission
and returned at the end, which indexes tensors of fixed per-request state (a recurrent or
convolution state of another mixer, a sampler's counters). This architecture's attention
keeps no such state, but the slot is still allocated, so that a part that does can be added
without touching this file.

The reference has none of this: one contiguous allocation per K and V for `max_batch` slots
(src/api.cu:1409-1411), a slot being reused by overwriting (2107-2123).
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np


class OutOfPages(RuntimeError):
    """A group's pool cannot cover the tokens asked for. Nothing was allocated."""


class OutOfStateSlots(RuntimeError):
    pass


class CacheError(RuntimeError):
    """Misuse: unknown or duplicate request, a page freed twice."""


# kind -> rule(group spec, position of the next query) -> [(lo, hi)): positions that no query from there on can see
RETENTION: Dict[str, Callable[["CacheGroupSpec", int], Sequence[Tuple[int, int]]]] = {}


def register_retention(kind: str, dead_ranges: Callable[["CacheGroupSpec", int], Sequence[Tuple[int, int]]]) -> None:
    """Adds a kind of cache group. `dead_ranges(spec, next_query_pos)` returns half-open ranges of positions whose
    entries no query at next_query_pos or later reads; a page that lies wholly inside one is given back."""
    RETENTION[kind] = dead_ranges


register_retention("full", lambda spec, q: ())
register_retention("window", lambda spec, q: ((0, max(0, q - spec.window + 1)),))


@dataclass(frozen=True)
class CacheGroupSpec:
    """What one group of layers needs. `n_layers` cache-owning layers share the group's block table; each keeps, per
    token, the `planes` (name, heads, width): by default keys and values of `kv_heads * head_dim` elements each.
    `extra` holds (key, value) pairs for a retention rule of another kind."""

    name: str
    kind: str  # a key of RETENTION: "full", "window", or one registered from outside
    n_layers: int
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    planes: Tuple[Tuple[str, int, int], ...] = ()
    extra: Tuple[Tuple[str, object], ...] = ()

    def __post_init__(self):
        if self.kind not in RETENTION:
            raise ValueError(f"cache group {self.name!r}: kind must be one of {sorted(RETENTION)}, got {self.kind!r}")
        if self.kind == "window" and self.window <= 0:
            raise ValueError(f"cache group {self.name!r}: a window group needs window > 0")
        if not self.planes:
            object.__setattr__(self, "planes", (("k", self.kv_heads, self.head_dim), ("v", self.kv_heads, self.head_dim)))
        names = [p[0] for p in self.planes]
        if len(set(names)) != len(names) or any(h <= 0 or d <= 0 for _, h, d in self.planes):
            raise ValueError(f"cache group {self.name!r}: planes need distinct names and positive sizes, got {self.planes}")

    def elements_per_token(self) -> int:
        return self.n_layers * sum(h * d for _, h, d in self.planes)


class PagePool:
    """Page ids 0..n-1 of one group; lowest free id first; every id is either free or held once."""

    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages))
        heapq.heapify(self._free)
        self._held = [False] * self.num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = heapq.heappop(self._free)
        self._held[p] = True
        return p

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or not self._held[page]:
            raise CacheError(f"page {page} is released but not held")
        self._held[page] = False
        heapq.heappush(self._free, page)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


class SlotPool:
    """State-slot ids 0..n-1, lowest free id first."""

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots))
        heapq.heapify(self._free)
        self._held = [False] * self.num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfStateSlots(f"all {self.num_slots} state slots are in use")
        s = heapq.heappop(self._free)
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._held[slot]:
            raise CacheError(f"state slot {slot} is released but not held")
        self._held[slot] = False
        heapq.heappush(self._free, slot)


@dataclass
class RequestCache:
    """What one live request holds: its length, its state slot, one block table per group."""

    request_id: object
    state_slot: int
    length: int = 0
    tables: List[List[int]] = field(default_factory=list)  # per group: logical page -> page id or -1
    fresh_slot: bool = True  # the state slot has not been zeroed on the device yet


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroupSpec], page_size: int, num_pages: Sequence[int] | int,
                 num_state_slots: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = int(page_size)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        if len(num_pages) != len(self.groups):
            raise ValueError("num_pages needs one entry per cache group")
        self.pools = [PagePool(n) for n in num_pages]
        self.slots = SlotPool(num_state_slots)
        self.requests: Dict[object, RequestCache] = {}

    # ---------------------------------------------------------------- requests
    def add_request(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        rc = RequestCache(request_id, self.slots.alloc(), 0, [[] for _ in self.groups])
        self.requests[request_id] = rc
        return rc

    def has_request(self, request_id) -> bool:
        return request_id in self.requests

    def get(self, request_id) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def free_request(self, request_id) -> None:
        """Give back every page and the state slot of a request that has ended."""
        rc = self.get(request_id)
        for g, table in enumerate(rc.tables):
            for p in table:
                if p >= 0:
                    self.pools[g].release(p)
        self.slots.release(rc.state_slot)
        del self.requests[request_id]

    # ---------------------------------------------------------------- pages
    def pages_needed(self, request_id, n_tokens: int) -> List[int]:
        """Per group: pages that appending n_tokens would take from the pool."""
        rc = self.requests.get(request_id)
        length = rc.length if rc else 0
        need = []
        for g in range(len(self.groups)):
            have = len(rc.tables[g]) if rc else 0
            total = -(-(length + n_tokens) // self.page_size)
            need.append(max(0, total - have))
        return need

    def can_append(self, request_id, n_tokens: int) -> bool:
        return all(n <= pool.free_count for n, pool in zip(self.pages_needed(request_id, n_tokens), self.pools))

    def append(self, request_id, n_tokens: int, as_arrays: bool = False) -> List[List[int]]:
        """Make room for positions [length, length + n_tokens) in every group and advance the
        length. Returns, per group, the cache slot (page id * page_size + offset) of each new
        position (lists; with as_arrays the maps of longer portions stay the integer arrays they
        were computed as). Raises OutOfPages, leaving everything as it was, if a pool is too small."""
        rc = self.get(request_id)
        need = self.pages_needed(request_id, n_tokens)
        for g, (n, pool) in enumerate(zip(need, self.pools)):
            if n > pool.free_count:
                raise OutOfPages(f"group {self.groups[g].name!r}: request {request_id!r} needs {n} more pages for "
                                 f"{n_tokens} tokens, {pool.free_count} of {pool.num_pages} are free")
        slot_maps = []
        for g, n in enumerate(need):
            table = rc.tables[g]
            for _ in range(n):
                table.append(self.pools[g].alloc())
            ps = self.page_size
            if n_tokens <= 8:
                slot_maps.append([table[p // ps] * ps + p % ps for p in range(rc.length, rc.length + n_tokens)])
            else:       # a prompt portion: the same in one numpy expression
                p = np.arange(rc.length, rc.length + n_tokens)
                first = rc.length // ps
                pages = np.asarray(table[first:(rc.length + n_tokens - 1) // ps + 1], dtype=np.int64)
                m = pages[p // ps - first] * ps + p % ps
                slot_maps.append(m if as_arrays else m.tolist())
        rc.length += n_tokens
        return slot_maps

    def release_behind_window(self, request_id) -> int:
        """After a step: give back the pages that, by the group's retention rule, no later token can see.
        The next query is at position `length`. Returns how many pages were released."""
        rc = self.get(request_id)
        released = 0
        ps = self.page_size
        for g, spec in enumerate(self.groups):
            table = rc.tables[g]
            for lo, hi in RETENTION[spec.kind](spec, rc.length):
                for lp in range(-(-lo // ps), min(hi // ps, len(table))):
                    if table[lp] >= 0:
                        self.pools[g].release(table[lp])
                        table[lp] = -1
                        released += 1
        return released

    # ---------------------------------------------------------------- views and checks
    def block_table(self, request_id, g: int) -> List[int]:
        return self.get(request_id).tables[g]

    def free_pages(self) -> List[int]:
        return [p.free_count for p in self.pools]

    def check(self) -> None:
        """Every page is free or held by exactly one request; every slot likewise. For tests."""
        for g, pool in enumerate(self.pools):
            owned: Dict[int, object] = {}
            for rid, rc in self.requests.items():
                for p in rc.tables[g]:
                    if p < 0:
                        continue
                    if p in owned:
                        raise CacheError(f"group {g}: page {p} is held by {owned[p]!r} and {rid!r}")
                    owned[p] = rid
            held = set(pool.held())
            if held != set(owned):
                raise CacheError(f"group {g}: pool holds {sorted(held)}, requests hold {sorted(owned)}")
            if len(held) + pool.free_count != pool.num_pages:
                raise CacheError(f"group {g}: {len(held)} held + {pool.free_count} free != {pool.num_pages}")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) + self.slots.free_count != self.slots.num_slots:
            raise CacheError("state slots are lost or held twice")
