"""Device storage of the cache and its grouping.

Layers whose mixers ask for the same thing (kv heads, head size, all keys or a window of them)
form a *group* with storage of its own: one key and one value pool
``[entries, pages, kv_heads, page_tokens, head_dim]`` shared by the group's entries, one page list
per sequence for the whole group.  Beside the pools each mixer that asks for it has a fixed-size
state block per slot, ``[num_slots + 1, *shape]`` (the last row is a spare for padded rows), zeroed when a slot is handed out; the architecture
built here asks for none, and the plumbing is exercised by a toy mixer in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVRequest, StateRequest
from .book import CacheBook, GroupGeometry


@dataclass
class CacheView:
    """What one schedule position sees of the cache."""

    group: int | None = None          # index of its kv group (None: no keys/values)
    k: torch.Tensor | None = None     # [pages, kv_heads, page_tokens, head_dim]
    v: torch.Tensor | None = None
    page_tokens: int = 0
    ring_tokens: int = 0              # 0: position p sits at element p; else at p % ring_tokens
    writable: bool = True             # False: this call reads an entry that another call writes
    state: torch.Tensor | None = None  # [num_slots + 1, *shape]; the last row belongs to no sequence (padded rows of a fixed-shape step)


@dataclass
class _Group:
    request: KVRequest
    owners: list[int]                 # schedule positions that own an entry, in order
    ring_tokens: int
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None


def round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class SequenceCache:
    """Slots, paged key/value pools per group, and per-slot state.

    ``requests[i]`` is what schedule position ``i`` asks for (``KVRequest``, ``StateRequest`` or
    None; or a list of them where the layer has several parts that keep something per sequence) and
    ``cache_of[i]`` the position whose entries it reads instead (or None).  ``view(i)`` gives one
    ``CacheView`` for a single request and a tuple of them, in the order asked, for a list.
    """

    def __init__(self, requests, cache_of, *, max_tokens: int, max_seq_len: int, dtype: torch.dtype,
                 device: torch.device, page_tokens: int = 64, chunk_tokens: int = 256,
                 num_slots: int | None = None, allocate: bool = True) -> None:
        self.page_tokens = page_tokens
        self.dtype = dtype
        self.device = device
        self.chunk_tokens = chunk_tokens
        self.max_seq_len = max_seq_len
        total_pages = max(1, round_up(max_tokens, page_tokens) // page_tokens)
        self.num_slots = num_slots if num_slots is not None else total_pages
        self.groups: list[_Group] = []
        self._entry_of: dict[tuple[int, int], tuple[int, int]] = {}     # (schedule position, request number) -> (group, entry)
        self._state_of: dict[tuple[int, int], torch.Tensor] = {}
        self._state_requests: dict[tuple[int, int], StateRequest] = {}
        self._cache_of = list(cache_of)
        self._counts: list[int | None] = []        # requests per position (None: a single request, viewed as one CacheView)
        for position, asked in enumerate(requests):
            several = isinstance(asked, (list, tuple))
            self._counts.append(len(asked) if several else None)
            if self._cache_of[position] is not None:
                continue
            for number, request in enumerate(asked if several else [asked]):
                if request is None:
                    continue
                key = (position, number)
                if isinstance(request, StateRequest):
                    self._state_requests[key] = request
                    continue
                for index, group in enumerate(self.groups):
                    if group.request == request:
                        break
                else:
                    ring = 0
                    if request.window:
                        ring = round_up(request.window + chunk_tokens - 1, page_tokens)
                    self.groups.append(_Group(request, [], ring))
                    index = len(self.groups) - 1
                self._entry_of[key] = (index, len(self.groups[index].owners))
                self.groups[index].owners.append(key)
        geometry = [GroupGeometry(total_pages, g.ring_tokens // page_tokens) for g in self.groups]
        self.book = CacheBook(self.num_slots, page_tokens, geometry, max_seq_len)
        self.has_window = any(g.ring_tokens for g in self.groups)
        # one page beyond the book's pool and one state row beyond the slots: padded rows of a fixed-shape decode
        # step read and write only these, never what a live sequence holds
        self.dummy_page = total_pages
        self.dummy_slot = self.num_slots
        if allocate:
            for group in self.groups:
                shape = (len(group.owners), total_pages + 1, group.request.kv_heads, page_tokens, group.request.head_dim)
                group.k = torch.zeros(shape, dtype=dtype, device=device)
                group.v = torch.zeros(shape, dtype=dtype, device=device)
            for key, request in self._state_requests.items():
                self._state_of[key] = torch.zeros((self.num_slots + 1, *request.shape), dtype=request.dtype, device=device)

    # ------------------------------------------------------------------ views
    def view(self, position: int):
        source = self._cache_of[position]
        owner = position if source is None else source
        count = self._counts[owner]
        views = []
        for number in range(1 if count is None else count):
            key = (owner, number)
            view = CacheView(page_tokens=self.page_tokens, writable=source is None)
            if key in self._entry_of:
                group_index, entry = self._entry_of[key]
                group = self.groups[group_index]
                view.group = group_index
                view.ring_tokens = group.ring_tokens
                if group.k is not None:
                    view.k, view.v = group.k[entry], group.v[entry]
            if key in self._state_of:
                view.state = self._state_of[key]
            views.append(view)
        return views[0] if count is None else tuple(views)

    # ------------------------------------------------------------------ slots
    def alloc(self) -> int:
        slot = self.book.alloc()
        for state in self._state_of.values():
            state[slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        self.book.free(slot)

    def max_blocks(self, group: int) -> int:
        ring = self.groups[group].ring_tokens
        return ring // self.page_tokens if ring else -(-self.max_seq_len // self.page_tokens)

    def bytes(self) -> int:
        total = 0
        for group in self.groups:
            if group.k is not None:
                total += 2 * group.k.numel() * group.k.element_size()
        for state in self._state_of.values():
            total += state.numel() * state.element_size()
        return total

    def token_bytes(self) -> int:
        """Bytes of keys and values one cached token occupies over all full-attention entries."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.owners) * g.request.kv_heads * g.request.head_dim * size for g in self.groups)
