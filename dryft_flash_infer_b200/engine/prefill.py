"""Short prompt steps as CUDA graphs.

A step of a few hundred tokens launches some three hundred kernels whose work on the
device takes less time than the host needs to launch them.  Such steps are laid out at
one of a few fixed shapes (16, 32 or 64 rows or a multiple of 128, sequences and wanted places
in powers of two; see ``StepContext``'s ``shape``), so that every step of a shape runs on the same
buffers, and the kernels of a shape are captured once and replayed.  What lies past a
step's own rows is computed and thrown away: it reaches no live page of the cache and no
other row, so it changes no result.  Steps that fit no shape (more than ``MAX_ROWS`` rows,
where the device is the slower side anyway, or many wanted places) run kernel by kernel.
"""

from __future__ import annotations

import torch

from .context import StepContext, StepEntry

ROW_UNIT = 128
SMALL_ROWS = 64        # the most rows the decode products take
MAX_ROWS = 1024
MAX_SEQS = 64          # of a shape, the spare one included
MAX_WANTED = 64
MAX_GRAPHS = 12


def _power_of_two(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


def shape_for(entries: list[StepEntry]) -> tuple[int, int, int] | None:
    """The padded shape ``(rows, sequences, wanted)`` of a step, or None if it runs as it is."""
    rows = sum(len(e.tokens) for e in entries)
    wanted = sum(len(e.want) for e in entries)
    if rows > MAX_ROWS or wanted == 0 or wanted > MAX_WANTED or len(entries) + 1 > MAX_SEQS:
        return None
    if all(len(e.tokens) == 1 for e in entries):
        return None            # decode steps have fixed buffers of their own
    # up to 64 rows the products run the decode kernels (which read the weights at a higher rate than the
    # library's 128-row tiles): such steps are padded to 16, 32 or 64 rows, not to 128
    padded = max(16, _power_of_two(rows)) if rows <= SMALL_ROWS else -(-rows // ROW_UNIT) * ROW_UNIT
    return (padded, _power_of_two(len(entries) + 1), _power_of_two(wanted))


class _Shape:
    """The fixed device buffer of one shape and, from its second use on, its graph."""

    def __init__(self, words: int, device):
        self.buffer = torch.zeros(words, dtype=torch.int32, device=device)
        self.uses = 0
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None


class PrefillGraphs:
    """Runs prompt steps that fit a shape; ``run`` returns None for the others."""

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self.widths = [max(1, -(-(g.ring_tokens or cache.max_context) // cache.page_size)) for g in cache.groups]
        self.shapes: dict[tuple[int, int, int], _Shape] = {}
        self.pool = None
        self.replays = 0

    def run(self, entries: list[StepEntry]):
        shape = shape_for(entries)
        if shape is None:
            return None
        held = self.shapes.pop(shape, None)
        if held is None:
            if len(self.shapes) >= MAX_GRAPHS:
                self.shapes.pop(next(iter(self.shapes)))        # the one whose last use is the longest ago
            rows, seqs, wanted = shape
            words = 3 * rows + 3 * seqs + (seqs + 1) + wanted + sum(seqs * w for w in self.widths) + 64
            held = _Shape(words, self.model.device)
        self.shapes[shape] = held                               # the dictionary keeps the order of last use
        ctx = StepContext(entries, self.cache, self.model.device, table_widths=self.widths, shape=shape,
                          into=held.buffer)
        held.uses += 1
        if held.uses == 1:
            # as it is: this use also sizes every scratch buffer and warms the library's products
            logits = self.model.forward(ctx, self.cache)
        else:
            if held.graph is None:
                torch.cuda.synchronize()
                if self.pool is None:
                    self.pool = torch.cuda.graph_pool_handle()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=self.pool):
                    held.logits = self.model.forward(ctx, self.cache)
                held.graph = graph
            held.graph.replay()
            self.replays += 1
            logits = held.logits
        # the caller keeps its logits while later steps reuse the buffers
        return logits[:ctx.own_wanted].clone()
