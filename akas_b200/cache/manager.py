"""The cache manager: pages of keys and values with a block table per request, and state slots.

kreasof-ai/akas owns persistent state by *slot*: per slot a contiguous key/value
cache of ``max_context`` tokens and the convolution history, zeroed at admission
and release (src/akas/execution/state.py:6-41, executor.py:75-88, 348-356;
layouts in src/akas/memory/layouts.py:8-66). Here a request owns

* a **slot** (0 .. max_requests-1) for state of fixed size: one row per slot in a
  tensor per state-holding layer, zeroed at admission; and
* in every **group** of paged layers, a list of **pages**. Layers with the same
  needs (all keys, or a window of the same length) form a group; a group has its
  own page numbers, free list and block tables, and each of its layers has its own
  pool of pages indexed by those numbers. Pages are taken when tokens are about to
  be written, given back when the request ends or, in a windowed group, when the
  window has passed them, and handed to later requests without being cleared: a
  key is reachable only through a block table and a position, so what an earlier
  owner left is never read (the reference argues the same for its slots).

All bookkeeping is host-side Python and needs no device (``storage=False``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..parts.base import PagedSpec, StateSpec


class OutOfPages(RuntimeError):
    """A group has too few free pages for the tokens that were to be written."""


class OutOfSlots(RuntimeError):
    """Every state slot is held by a live request."""


class PageAllocator:
    """Free list of one group's pages. A page is free or held by exactly one request."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() hands out low numbers first
        self._held = [False] * num_pages

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        self._held[page] = True
        return page

    def give(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise RuntimeError(f"page {page} is given back but is not held")
        self._held[page] = False
        self._free.append(page)


class PagedCache:
    """What a paged mixer gets: its own pools (attributes named as its spec named them, ``None`` without storage), the
    group whose block table addresses them, and that group's page size."""

    def __init__(self, pools: Dict[str, Optional[torch.Tensor]], group: int, page_size: int, spec: PagedSpec):
        self.pools, self.group, self.page_size, self.spec = pools, group, page_size, spec

    def __getattr__(self, name):
        pools = self.__dict__.get("pools", {})
        if name in pools:
            return pools[name]
        raise AttributeError(name)


@dataclass
class StateCache:
    """What a stateful mixer gets: ``state[slot]`` is the row of the request in that slot."""

    state: Optional[torch.Tensor]
    spec: StateSpec = None


@dataclass
class _Group:
    window: Optional[int]
    allocator: PageAllocator
    page_size: int = 0
    max_blocks: int = 0  # columns of this group's block table: the pages a request of full context holds
    blocks: Dict[Hashable, List[int]] = field(default_factory=dict)  # request -> page per block, -1 once released


@dataclass
class _Request:
    slot: int
    length: int = 0  # tokens written so far
    reserved: int = 0  # tokens that have pages


class CacheManager:
    def __init__(self, cache_specs: Sequence, page_size: int, pool_tokens: int, max_requests: int,
                 context: int, dtype=torch.float32, device="cpu", storage: bool = True):
        """``cache_specs``: for each schedule entry the spec its mixer asked for, or None.

        Every group gets ``pool_tokens // its page size`` pages (the engine's ``page_size`` unless the group's
        specs name their own); a request may hold up to ``context`` tokens, so a group's block table has
        ``ceil(context / its page size)`` columns.
        """
        if page_size < 1 or pool_tokens < page_size:
            raise ValueError(f"pool of {pool_tokens} tokens holds no page of {page_size}")
        self.page_size = page_size
        self.num_pages = pool_tokens // page_size
        self.max_requests = max_requests
        self.context = context
        self.max_blocks = -(-context // page_size)
        self.groups: List[_Group] = []
        self.views: List[Optional[object]] = []
        self.state_tensors: List[torch.Tensor] = []  # [layers of one state shape, slots, *shape]: zeroed per slot in one go
        self._group_of: Dict[tuple, int] = {}  # a spec's paging() -> group
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self.peak_pages = 0
        # states of one shape and type share an allocation, so that a slot is zeroed across layers by one launch
        backing: Dict[tuple, torch.Tensor] = {}
        taken: Dict[tuple, int] = {}
        if storage:
            count: Dict[tuple, int] = {}
            for spec in cache_specs:
                if isinstance(spec, StateSpec):
                    key = (tuple(spec.shape), spec.dtype)
                    count[key] = count.get(key, 0) + 1
            for key, layers in count.items():
                backing[key] = torch.zeros((layers, max_requests, *key[0]), dtype=key[1], device=device)
                taken[key] = 0
                self.state_tensors.append(backing[key])
        for spec in cache_specs:
            if spec is None:
                self.views.append(None)
            elif isinstance(spec, PagedSpec):
                size = spec.page_size or page_size
                if size < 1 or pool_tokens < size:
                    raise ValueError(f"pool of {pool_tokens} tokens holds no page of {size}")
                gid = self._group_of.get(spec.paging())
                if gid is None:
                    gid = len(self.groups)
                    self._group_of[spec.paging()] = gid
                    self.groups.append(_Group(spec.window, PageAllocator(pool_tokens // size), page_size=size,
                                              max_blocks=-(-context // size)))
                pools = {name: None for name in spec.pools(size)}
                if storage:
                    pages = self.groups[gid].allocator.num_pages
                    pools = {name: torch.zeros((pages, *shape), dtype=spec.dtype or dtype, device=device)
                             for name, shape in spec.pools(size).items()}
                self.views.append(PagedCache(pools, gid, size, spec))
            elif isinstance(spec, StateSpec):
                state = None
                if storage:
                    key = (tuple(spec.shape), spec.dtype)
                    state = backing[key][taken[key]]
                    taken[key] += 1
                self.views.append(StateCache(state, spec))
            else:
                raise TypeError(f"unknown cache spec {spec!r}")

    # ------------------------------------------------------------------ requests

    def __contains__(self, request) -> bool:
        return request in self._requests

    def live(self) -> List[Hashable]:
        return list(self._requests)

    def slot(self, request) -> int:
        return self._requests[request].slot

    def length(self, request) -> int:
        return self._requests[request].length

    @property
    def table_widths(self) -> List[int]:
        """Columns of each group's block table."""
        return [g.max_blocks for g in self.groups]

    def capacity_tokens(self) -> int:
        """The most tokens one request can hold when it has the pool to itself (a windowed group gives pages back as
        it goes, so only groups that keep everything bound it)."""
        full = [g.allocator.num_pages * g.page_size for g in self.groups if g.window is None]
        return min(full, default=self.context)

    def fits(self, tokens: int) -> bool:
        """Whether every group has free pages for the first ``tokens`` tokens of a request that holds none yet."""
        return all(-(-tokens // g.page_size) <= g.allocator.free for g in self.groups)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.free if self.groups else self.num_pages

    def min_free_pages(self) -> int:
        return min((g.allocator.free for g in self.groups), default=self.num_pages)

    def admit(self, request, zero=None) -> int:
        """Gives ``request`` a slot and zeroes its state rows (by ``zero(tensor, slot)`` if given, for a tensor
        ``[layers, slots, ...]``)."""
        if request in self._requests:
            raise RuntimeError(f"request {request!r} is already admitted")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} slots are held")
        slot = self._free_slots.pop()
        self._requests[request] = _Request(slot)
        for group in self.groups:
            group.blocks[request] = []
        for state in self.state_tensors:
            if zero is not None:
                zero(state, slot)
            else:
                state[:, slot].zero_()
        return slot

    def pages_needed(self, request, tokens: int) -> List[int]:
        """Pages each group lacks before ``tokens`` more tokens of ``request`` can be written."""
        req = self._requests[request]
        end = req.length + tokens
        return [max(0, -(-end // group.page_size) - len(group.blocks[request])) for group in self.groups]

    def room(self, request) -> int:
        """How many more tokens of ``request`` could be reserved now: the rest of its last page plus the
        free pages of the fullest group, and never past the context."""
        req = self._requests[request]
        if not self.groups:
            return self.context - req.length
        room = min(max(0, len(g.blocks[request]) * g.page_size - req.length) + g.allocator.free * g.page_size
                   for g in self.groups)
        return min(room, self.context - req.length)

    def reserve(self, request, tokens: int) -> None:
        """Takes pages in every group for the next ``tokens`` positions; all groups or none."""
        req = self._requests[request]
        if req.length + tokens <= req.reserved:
            return  # already covered (the scheduler reserves when it plans, the step function when it runs)
        if req.length + tokens > self.context:
            raise ValueError(f"request {request!r}: {req.length + tokens} tokens exceed the context of {self.context}")
        need = self.pages_needed(request, tokens)
        for group, n in zip(self.groups, need):
            if n > group.allocator.free:
                raise OutOfPages(f"{n} pages wanted, {group.allocator.free} free (window {group.window})")
        for group, n in zip(self.groups, need):
            group.blocks[request].extend(group.allocator.take() for _ in range(n))
        req.reserved = max(req.reserved, req.length + tokens)
        used = max((g.allocator.num_pages - g.allocator.free for g in self.groups), default=0)
        self.peak_pages = max(self.peak_pages, used)

    def advance(self, request, tokens: int) -> None:
        """Records that ``tokens`` more positions are written; gives back pages a window has passed."""
        req = self._requests[request]
        if req.length + tokens > req.reserved:
            raise RuntimeError(f"request {request!r} advances past its reserved pages")
        req.length += tokens
        for group in self.groups:
            if group.window is None:
                continue
            # the next query sits at position `length` and sees keys >= length - window + 1
            first_needed = req.length - group.window + 1
            blocks = group.blocks[request]
            for b in range(min(len(blocks), max(0, first_needed) // group.page_size)):
                if blocks[b] >= 0:
                    group.allocator.give(blocks[b])
                    blocks[b] = -1

    def release(self, request) -> None:
        """The request ends: its pages and its slot go back."""
        req = self._requests.pop(request)
        for group in self.groups:
            for page in group.blocks.pop(request):
                if page >= 0:
                    group.allocator.give(page)
        self._free_slots.append(req.slot)

    def blocks(self, request, group: int) -> List[int]:
        return self.groups[group].blocks[request]

    # ------------------------------------------------------------------ self-check

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost or shared. Raises AssertionError."""
        for gid, group in enumerate(self.groups):
            held = [p for blocks in group.blocks.values() for p in blocks if p >= 0]
            free = group.allocator._free
            assert len(set(held)) == len(held), f"group {gid}: a page is held twice"
            assert len(set(free)) == len(free), f"group {gid}: a page is free twice"
            assert not set(held) & set(free), f"group {gid}: a page is both held and free"
            assert len(held) + len(free) == group.allocator.num_pages, f"group {gid}: a page is lost"
            assert set(group.blocks) == set(self._requests), f"group {gid}: block lists and requests differ"
        slots = [r.slot for r in self._requests.values()]
        assert len(set(slots)) == len(slots) and not set(slots) & set(self._free_slots), "a slot is shared"
        assert len(slots) + len(self._free_slots) == self.max_requests, "a slot is lost"
