"""Host-side bookkeeping of the cache: which slot and which pages each sequence holds.

Pure Python, no device work: the storage that the ids index lives in
``cache/storage.py``.  A *slot* stands for one live sequence; a *page* is room for
``page_size`` tokens of keys and values in every cache entry of one group.
Slots and pages return to their free lists when a sequence ends and are handed
out again to later sequences.
"""

from __future__ import annotations

import heapq


class CacheError(RuntimeError):
    """The cache cannot do what was asked: out of slots or pages, or a misuse such as
    freeing a slot twice.  The message says which."""


class FreeList:
    """Ids ``first .. first+count-1``, handed out lowest-first, each held at most once."""

    def __init__(self, count: int, first: int = 0, what: str = "id"):
        self.what = what
        self._all = range(first, first + count)
        self._free = list(self._all)          # a heap: the lowest free id is taken next
        self._held: set[int] = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"out of {self.what}s: all {len(self._all)} are held")
        item = heapq.heappop(self._free)
        self._held.add(item)
        return item

    def give_back(self, item: int) -> None:
        if item not in self._held:
            state = "is already free" if item in self._all else "was never handed out"
            raise CacheError(f"{self.what} {item} {state}")
        self._held.remove(item)
        # lowest id first keeps reuse predictable (and exercised: a freed id is the next one taken)
        heapq.heappush(self._free, item)

    def check(self) -> None:
        """No id lost and none held twice."""
        free = set(self._free)
        assert len(free) == len(self._free), f"a {self.what} is on the free list twice"
        assert not (free & self._held), f"a {self.what} is both free and held"
        assert free | self._held == set(self._all), f"a {self.what} was lost"


class GroupPages:
    """The pages of one cache group: a pool, and for each slot the pages it holds in order.

    A group with a window keeps a fixed ring of ``ring_tokens`` token places per
    sequence (position ``p`` lives at place ``p % ring_tokens``), taken whole when the
    slot is taken.  A group without window (``ring_tokens`` = 0) grows page by page
    with the sequence.  Page 0 is never handed out: block tables are padded with it.
    """

    def __init__(self, n_pages: int, page_size: int, ring_tokens: int = 0, name: str = "group"):
        if ring_tokens % page_size:
            raise ValueError("ring_tokens must be a multiple of the page size")
        self.page_size, self.ring_tokens, self.name = page_size, ring_tokens, name
        self.pool = FreeList(n_pages - 1, first=1, what=f"page of {name}")
        self.pages_of: dict[int, list[int]] = {}

    def pages_for(self, n_tokens: int) -> int:
        if self.ring_tokens:
            return self.ring_tokens // self.page_size
        return -(-n_tokens // self.page_size)

    def open_slot(self, slot: int) -> None:
        if slot in self.pages_of:
            raise CacheError(f"slot {slot} already holds pages of {self.name}")
        self.pages_of[slot] = []
        if self.ring_tokens:
            self.reserve(slot, self.ring_tokens)

    def reserve(self, slot: int, n_tokens: int) -> bool:
        """Makes sure ``slot`` has room for ``n_tokens`` tokens; True if pages were added."""
        pages = self.pages_of[slot]
        want = self.pages_for(n_tokens)
        if want - len(pages) > self.pool.free:
            raise CacheError(
                f"out of cache pages in {self.name}: slot {slot} needs {want - len(pages)} more pages of "
                f"{self.page_size} tokens, {self.pool.free} are free (raise max_tokens)")
        grew = False
        while len(pages) < want:
            pages.append(self.pool.take())
            grew = True
        return grew

    def close_slot(self, slot: int) -> None:
        if slot not in self.pages_of:
            raise CacheError(f"slot {slot} holds no pages of {self.name} (freed twice?)")
        for page in self.pages_of.pop(slot):
            self.pool.give_back(page)

    def check(self) -> None:
        self.pool.check()
        seen: set[int] = set()
        for slot, pages in self.pages_of.items():
            for page in pages:
                assert page not in seen, f"page {page} of {self.name} is held by two slots"
                seen.add(page)
        assert len(seen) == self.pool.held, f"pages of {self.name} held by no slot"


class SlotBook:
    """Slots, their lengths, and their pages in every group."""

    def __init__(self, n_slots: int, groups: list[GroupPages], max_context: int):
        self.slots = FreeList(n_slots, what="slot")
        self.groups = groups
        self.max_context = max_context
        self.length: dict[int, int] = {}

    def open(self) -> int:
        slot = self.slots.take()
        try:
            for group in self.groups:
                group.open_slot(slot)
        except CacheError:
            for group in self.groups:
                if slot in group.pages_of:
                    group.close_slot(slot)
            self.slots.give_back(slot)
            raise
        self.length[slot] = 0
        return slot

    def close(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open (freed twice?)")
        for group in self.groups:
            group.close_slot(slot)
        del self.length[slot]
        self.slots.give_back(slot)

    def reserve(self, slot: int, new_tokens: int) -> None:
        """Room for ``new_tokens`` more tokens in ``slot``; the length itself moves in ``advance``."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open")
        total = self.length[slot] + new_tokens
        if total > self.max_context:
            raise CacheError(f"slot {slot}: {total} tokens exceed max_context {self.max_context}")
        for group in self.groups:
            group.reserve(slot, total)

    def advance(self, slot: int, new_tokens: int) -> None:
        self.length[slot] += new_tokens

    def check(self) -> None:
        self.slots.check()
        assert set(self.length) == self.slots._held, "open slots and held slots differ"
        for group in self.groups:
            group.check()
            assert set(group.pages_of) == set(self.length), f"{group.name} has pages of a closed slot"
