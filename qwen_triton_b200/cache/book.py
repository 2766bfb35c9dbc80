"""Host-side bookkeeping of the cache: which sequence holds which slot and which pages.

A *slot* belongs to one live sequence: it indexes the fixed-size per-sequence state and carries
the sequence's length and, for each cache group, the list of pages that hold its keys and values.
Pages are ``page_tokens`` positions long.  A group that keeps all keys takes pages as the sequence
grows; a group that keeps a window of them takes at most ``ring_pages`` and reuses them as a ring.
Slots and pages go back to their free lists when the sequence ends and are handed out again.

No device memory is touched here, so the invariants (no slot or page lost, held twice or freed
twice) can be checked without a GPU.  The reference keeps one length for the whole batch and grows
its tensors by reallocation (qwen_triton/modules/cache.py:21-65).
"""
from __future__ import annotations

from dataclasses import dataclass, field


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot or page is left for the request."""


@dataclass(frozen=True)
class GroupGeometry:
    """One cache group as the book sees it: its page pool and, for a windowed group, its ring."""

    num_pages: int
    ring_pages: int = 0      # 0: keeps every position; else pages of the ring a sequence cycles through


@dataclass
class _Slot:
    length: int = 0
    pages: list[list[int]] = field(default_factory=list)   # per group


class CacheBook:
    def __init__(self, num_slots: int, page_tokens: int, groups: list[GroupGeometry], max_seq_len: int) -> None:
        if num_slots <= 0 or page_tokens <= 0 or max_seq_len <= 0:
            raise ValueError("num_slots, page_tokens and max_seq_len must be positive")
        self.num_slots = num_slots
        self.page_tokens = page_tokens
        self.groups = list(groups)
        self.max_seq_len = max_seq_len
        self._free_slots = list(range(num_slots - 1, -1, -1))         # pop() hands out the lowest number first
        self._free_pages = [list(range(g.num_pages - 1, -1, -1)) for g in self.groups]
        self._live: dict[int, _Slot] = {}

    # ------------------------------------------------------------------ slots
    def alloc(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.num_slots} sequence slots are in use")
        slot = self._free_slots.pop()
        self._live[slot] = _Slot(0, [[] for _ in self.groups])
        return slot

    def free(self, slot: int) -> None:
        entry = self._live.pop(slot, None)
        if entry is None:
            raise CacheError(f"slot {slot} is not in use (freed twice, or never allocated)")
        for group, pages in enumerate(entry.pages):
            self._free_pages[group].extend(reversed(pages))
        self._free_slots.append(slot)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    def live_slots(self) -> list[int]:
        return sorted(self._live)

    def length(self, slot: int) -> int:
        return self._entry(slot).length

    def _entry(self, slot: int) -> _Slot:
        try:
            return self._live[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not in use") from None

    # ------------------------------------------------------------------ pages
    def pages_needed(self, group: int, length: int) -> int:
        pages = -(-length // self.page_tokens)
        ring = self.groups[group].ring_pages
        return min(pages, ring) if ring else pages

    def can_hold(self, lengths_by_slot: dict[int, int]) -> bool:
        """Whether every slot can grow to the given length at once."""
        for group in range(len(self.groups)):
            extra = 0
            for slot, length in lengths_by_slot.items():
                extra += max(0, self.pages_needed(group, length) - len(self._entry(slot).pages[group]))
            if extra > len(self._free_pages[group]):
                return False
        return True

    def extend(self, slot: int, new_length: int) -> None:
        """Make room for positions below ``new_length`` and record the new length."""
        entry = self._entry(slot)
        if new_length < entry.length:
            raise CacheError(f"slot {slot}: a sequence cannot shrink ({entry.length} -> {new_length})")
        if new_length > self.max_seq_len:
            raise CacheFull(f"slot {slot}: {new_length} tokens exceed the longest sequence the cache holds ({self.max_seq_len})")
        wanted = [self.pages_needed(g, new_length) - len(entry.pages[g]) for g in range(len(self.groups))]
        for group, count in enumerate(wanted):
            if count > len(self._free_pages[group]):
                raise CacheFull(f"cache group {group}: {count} more pages needed, {len(self._free_pages[group])} free")
        for group, count in enumerate(wanted):
            for _ in range(max(0, count)):
                entry.pages[group].append(self._free_pages[group].pop())
        entry.length = new_length

    def pages(self, slot: int, group: int) -> list[int]:
        return self._entry(slot).pages[group]

    def free_pages(self, group: int) -> int:
        return len(self._free_pages[group])

    def free_slot_count(self) -> int:
        return len(self._free_slots)

    # ------------------------------------------------------------------ checks
    def check(self) -> None:
        """Raise if a slot or page is lost or held twice."""
        slots = self._free_slots + list(self._live)
        if sorted(slots) != list(range(self.num_slots)):
            raise CacheError(f"slot accounting is broken: {sorted(slots)}")
        for group, geometry in enumerate(self.groups):
            held = [p for entry in self._live.values() for p in entry.pages[group]]
            everything = self._free_pages[group] + held
            if sorted(everything) != list(range(geometry.num_pages)):
                raise CacheError(f"page accounting of group {group} is broken")
