"""Device storage of the cache and the per-sequence state, laid out for the kernels.

Cache entries (one per schedule entry that writes keys and values) with the same
need (heads, head size, window) form a *group* with storage of its own:

    k, v : [entries, pages, kv_heads, page_size, head_dim]

so that a (page, head) block is ``page_size * head_dim`` contiguous elements: one
TMA box or a run of 16-byte loads for attention.  A sequence's pages are listed in
a block table ``[sequence, page index] -> page``; position ``p`` of a sequence lives
at place ``p`` (or ``p % ring_tokens`` in a group with a window), i.e. in page
``table[place // page_size]`` at row ``place % page_size``.

Beside the groups, every schedule entry whose mixer asks for it has a fixed-size
state per slot, ``[slots, *shape]``, in the dtype the mixer names (float32 or bfloat16),
set to the mixer's start value when a slot is opened.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVNeed, StateNeed
from .allocator import GroupPages, SlotBook

PAGE_SIZE = 64
_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@dataclass
class CacheGroup:
    need: KVNeed
    cache_ids: list[int]
    pages: GroupPages
    k: torch.Tensor
    v: torch.Tensor

    @property
    def ring_tokens(self) -> int:
        return self.pages.ring_tokens


@dataclass
class LayerCache:
    """What one mixer application sees of the cache during a step."""

    k: torch.Tensor            # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # int32 [sequences, table_width], of this step's sequences
    page_size: int
    ring_tokens: int
    writes: bool


def round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


class SequenceCache:
    """All groups, the slot book and the state areas of one engine."""

    def __init__(self, needs: dict[int, KVNeed], state_needs: dict[int, StateNeed], *, max_tokens: int,
                 max_seqs: int, max_context: int, step_tokens: int, dtype: torch.dtype, device):
        """``needs`` maps a cache id to its need; ``state_needs`` a schedule position to its state.

        ``max_tokens`` is the number of token places (each sequence rounded up to a
        page) that live sequences may hold together; ``step_tokens`` is the most
        tokens one step gives one sequence, which a ring has to hold beside its window.
        """
        self.page_size = PAGE_SIZE
        self.max_tokens, self.max_seqs, self.max_context = max_tokens, max_seqs, max_context
        self.dtype, self.device = dtype, device
        by_need: dict[KVNeed, list[int]] = {}
        for cache_id in sorted(needs):
            by_need.setdefault(needs[cache_id], []).append(cache_id)
        self.groups: list[CacheGroup] = []
        self.group_of: dict[int, tuple[int, int]] = {}
        for index, (need, ids) in enumerate(by_need.items()):
            if need.window:
                ring = round_up(need.window + step_tokens - 1, PAGE_SIZE)
                n_pages = 1 + max_seqs * (ring // PAGE_SIZE)
            else:
                ring = 0
                n_pages = 1 + round_up(max_tokens, PAGE_SIZE) // PAGE_SIZE
            pages = GroupPages(n_pages, PAGE_SIZE, ring, name=f"cache group {index}")
            shape = (len(ids), n_pages, need.n_kv_heads, PAGE_SIZE, need.head_dim)
            group = CacheGroup(need, ids, pages,
                               torch.zeros(shape, dtype=dtype, device=device),
                               torch.zeros(shape, dtype=dtype, device=device))
            self.groups.append(group)
            for position, cache_id in enumerate(ids):
                self.group_of[cache_id] = (index, position)
        self.book = SlotBook(max_seqs, [g.pages for g in self.groups], max_context)
        #: a slot that no sequence ever holds: the state of places that only fill a step's buffers (one row
        #: more in every state area, which nothing reads for a result)
        self.spare_slot = max_seqs
        self.state: dict[int, torch.Tensor] = {}
        self.state_init: dict[int, float] = {}
        for position, need in state_needs.items():
            if need.dtype not in _STATE_DTYPES:
                raise ValueError(f"a state is held in one of {sorted(_STATE_DTYPES)}, not {need.dtype!r}")
            self.state[position] = torch.full((max_seqs + 1,) + tuple(need.shape), float(need.init),
                                              dtype=_STATE_DTYPES[need.dtype], device=device)
            self.state_init[position] = float(need.init)

    # ------------------------------------------------------------------ slots
    def open_slot(self) -> int:
        slot = self.book.open()
        for position, area in self.state.items():
            area[slot].fill_(self.state_init[position])        # a slot used again starts as a new one does
        return slot

    def close_slot(self, slot: int) -> None:
        self.book.close(slot)

    def length(self, slot: int) -> int:
        return self.book.length[slot]

    @property
    def live_slots(self) -> int:
        return self.book.slots.held

    # ------------------------------------------------------------------ views
    def table_width(self, slots: list[int], group: int, fixed: int | None = None) -> int:
        pages = self.groups[group].pages
        width = max((len(pages.pages_of[s]) for s in slots), default=1)
        if fixed is not None:
            if width > fixed:
                raise ValueError("block table wider than the fixed width")
            return fixed
        return max(1, round_up(width, 4))

    def fill_block_table(self, out, slots: list[int], group: int, width: int) -> None:
        """Writes the ``[len(slots), width]`` table of ``group`` into the int32 array ``out``."""
        pages = self.groups[group].pages
        for row, slot in enumerate(slots):
            held = pages.pages_of[slot]
            out[row, :len(held)] = held
            out[row, len(held):] = 0

    def layer_view(self, cache_id: int, tables: list[torch.Tensor], writes: bool) -> LayerCache:
        group_index, position = self.group_of[cache_id]
        group = self.groups[group_index]
        return LayerCache(group.k[position], group.v[position], tables[group_index],
                          self.page_size, group.ring_tokens, writes)

    def bytes(self) -> int:
        return sum(g.k.numel() * g.k.element_size() * 2 for g in self.groups) + \
            sum(a.numel() * a.element_size() for a in self.state.values())
