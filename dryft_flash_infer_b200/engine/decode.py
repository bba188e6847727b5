"""The decode step on fixed device addresses, captured in a CUDA graph.

A decode step gives every sequence of a batch one token.  Its shapes depend only on
the number of sequences, so its buffers can stay where they are from step to step: the
step's numbers (positions, block tables, random numbers for sampling) are written into
one fixed device buffer before each step, the tokens are left there by the sampler of
the step before, and the kernels between are replayed as one CUDA graph, as the
reference replays its decode step (engine/engine.py:835-863, :1031-1049).  The same
code runs without a graph when graphs are switched off or a mixer cannot be captured.
"""

from __future__ import annotations

import os

import numpy as np
import torch

from ..ops import kernels
from ..sampling import SamplingParams, uniform_for


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class DecodeBatch:
    """Fixed buffers (and the graph) for decode steps of up to ``n`` sequences.

    It looks like a ``StepContext`` to the model: the same attributes, all views of one
    device buffer.  ``run`` refreshes the numbers that change and runs one step; the
    chosen tokens stay on the device as the next step's input and come back as a list.

    A step of fewer than ``n`` sequences fills the places past its own with sequences of one token at
    position 0 whose block tables name the null page only and whose state is the cache's spare slot:
    they cost a row of every product and a page of attention, reach nothing that lives, and what is
    chosen for them is thrown away.  So a live set that shrinks by a sequence keeps its buffers and its
    graph instead of running a step launch by launch and capturing a graph for every size on its way down.

    The attention kernel chooses its launch shape by how long a sequence may get (``max_kv_len``), and a
    graph holds the shape it was captured with.  The host knows every sequence's length, so a step says the
    smallest of ``kernels.DECODE_KV_STEPS`` that covers its longest sequence, and the batch keeps a graph for
    each limit it has met: all on the same buffers, so the tokens stay where they are when a batch grows
    past a limit.
    """

    all_decode = True
    wants_every_row = True
    max_q_len = 1
    upcoming = None          # as in StepContext: what the step streams after the part that is running
    decode_plans = None      # as in StepContext: what the kernels of one pass share between layers

    def __init__(self, model, cache, n: int, table_widths: list[int], max_context: int, temperature: float,
                 use_graph: bool):
        self.model, self.cache, self.n = model, cache, n
        self.n_seqs = self.n_rows = self.n_wanted = n
        self.table_widths = table_widths
        self.temperature = temperature
        self.use_graph = use_graph
        self.q_lens = [1] * n
        self.max_context = max_context
        self.max_kv_len = max_context     # of the step being launched: see ``launch``
        device = model.device
        sections = {"tokens": n, "row_seq": n, "row_pos": n, "seq_start": n, "seq_qlen": n, "seq_slot": n,
                    "cu_rows": n + 1, "wanted_rows": n, "uniforms": n}
        for g, width in enumerate(table_widths):
            sections[f"table{g}"] = n * width
        self.offsets, total = {}, 0
        for name, size in sections.items():
            self.offsets[name] = total
            total += _pad4(size)
        # A step's numbers travel through pinned staging buffers used in turn: the copy to the device is
        # asynchronous, and the next step (launched before this one's tokens are read) must not rewrite a
        # buffer whose copy has not run yet.  Each buffer has an event recorded after its copy.
        self.staging = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.staging_np = [t.numpy() for t in self.staging]
        self.tokens_staging = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.staging_event: list[torch.cuda.Event | None] = [None, None]
        self.device_buffer = torch.zeros(total, dtype=torch.int32, device=device)
        # results come back through two pinned buffers in turn, so that the host can read one step's
        # tokens while the next step is already running; the kernels' status words ride along
        self.result_host = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.status_host = [torch.zeros(kernels.STATUS_WORDS, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.status_device = kernels.status_words(device)
        self.result_event = [torch.cuda.Event() for _ in range(2)]
        self.live_of = [0, 0]             # sequences of the steps whose results the two buffers hold
        self.launched = 0
        #: float32 logits ``[n, vocab]`` of the step launched last (a fixed buffer once the graph exists)
        self.logits: torch.Tensor | None = None

        def dev(name, size):
            return self.device_buffer[self.offsets[name]: self.offsets[name] + size]

        self.tokens, self.row_seq, self.row_pos = dev("tokens", n), dev("row_seq", n), dev("row_pos", n)
        self.seq_start, self.seq_qlen, self.seq_slot = dev("seq_start", n), dev("seq_qlen", n), dev("seq_slot", n)
        self.cu_rows, self.wanted_rows = dev("cu_rows", n + 1), dev("wanted_rows", n)
        self.uniforms = dev("uniforms", n).view(torch.float32)
        self.block_tables = [dev(f"table{g}", n * w).view(n, w) for g, w in enumerate(table_widths)]
        for h in self.staging_np:
            h[self.offsets["row_seq"]: self.offsets["row_seq"] + n] = np.arange(n)
            h[self.offsets["seq_qlen"]: self.offsets["seq_qlen"] + n] = 1
            h[self.offsets["cu_rows"]: self.offsets["cu_rows"] + n + 1] = np.arange(n + 1)
            h[self.offsets["wanted_rows"]: self.offsets["wanted_rows"] + n] = np.arange(n)
        self.first_refreshed = self.offsets["row_seq"]
        self.h2d_bytes_per_step = (total - self.first_refreshed) * 4
        self.graph = None                 # of the limit used last: None (never run), False (run once), or the graph
        self.graphs: dict[int, tuple] = {}          # kv limit -> (graph or False, its logits)
        self.slots: list[int] = []
        self.starts: list[int] = []
        self.live = 0                     # sequences of the step launched last (the rest of the n places are filling)
        self.launches_per_step = 0
        self.last_out: list[int] | None = None

    def _body(self) -> None:
        logits = self.logits = self.model.forward(self, self.cache)
        if self.temperature == 0.0:
            kernels.argmax(logits, out=self.tokens)
        else:
            kernels.sample_temperature(logits, self.uniforms, self.temperature, out=self.tokens)

    def _refresh(self, slots: list[int], tokens: list[int] | None, uniforms) -> None:
        turn = self.launched & 1
        if self.staging_event[turn] is not None:
            self.staging_event[turn].synchronize()          # the copy that last read this buffer has run
        if tokens is not None:
            self.tokens_staging[turn][: len(tokens)] = torch.tensor(tokens, dtype=torch.int32)
            self.tokens_staging[turn][len(tokens):] = 0
            self.tokens.copy_(self.tokens_staging[turn], non_blocking=True)
        n, h, off = self.n, self.staging_np[turn], self.offsets
        live = self.live = len(slots)
        filling = n - live
        starts = [self.cache.length(s) for s in slots]
        # as a StepContext shows them, the filling included: its sequences sit at position 0 of the spare slot
        self.slots = slots + [self.cache.spare_slot] * filling
        self.starts = starts = starts + [0] * filling
        h[off["row_pos"]: off["row_pos"] + n] = starts
        h[off["seq_start"]: off["seq_start"] + n] = starts
        h[off["seq_slot"]: off["seq_slot"] + n] = self.slots
        if uniforms is not None:
            h[off["uniforms"]: off["uniforms"] + live] = np.asarray(uniforms, dtype=np.float32).view(np.int32)
            h[off["uniforms"] + live: off["uniforms"] + n] = 0
        for g, width in enumerate(self.table_widths):
            table = h[off[f"table{g}"]: off[f"table{g}"] + n * width].reshape(n, width)
            self.cache.fill_block_table(table[:live], slots, g, width)
            table[live:] = 0                                   # the null page
        first = self.first_refreshed
        self.device_buffer[first:].copy_(self.staging[turn][first:], non_blocking=True)
        if self.staging_event[turn] is None:
            self.staging_event[turn] = torch.cuda.Event()
        self.staging_event[turn].record()

    def launch(self, slots: list[int], tokens: list[int] | None, uniforms=None) -> int:
        """Starts one decode step for ``slots`` and returns a ticket for ``fetch``.  ``tokens`` None
        means: the tokens the last step chose (they are still on the device)."""
        book = self.cache.book
        for slot in slots:
            book.reserve(slot, 1)
        self._refresh(slots, tokens, uniforms)
        limit = self.max_kv_len = kernels.decode_kv_limit(max(self.starts) + 1, self.max_context)
        held = self.graphs.get(limit)
        if not self.use_graph:
            self._body()
        elif held is None:
            # the first step under a limit runs as it is (it also sizes every scratch buffer); the second is captured
            before = kernels.LAUNCHES
            self._body()
            self.launches_per_step = kernels.LAUNCHES - before
            self.graphs[limit] = (False, None)
            self.graph = False
        elif held[0] is False:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._body()
            # capturing does not run the kernels: replay once for this step
            graph.replay()
            self.graphs[limit] = (graph, self.logits)
            self.graph = graph
        else:
            self.graph, self.logits = held
            self.graph.replay()
        for slot in slots:
            book.advance(slot, 1)
        ticket = self.launched
        self.launched += 1
        self.live_of[ticket & 1] = len(slots)
        self.result_host[ticket & 1].copy_(self.tokens, non_blocking=True)
        self.status_host[ticket & 1].copy_(self.status_device, non_blocking=True)
        self.result_event[ticket & 1].record()
        return ticket

    def fetch(self, ticket: int) -> list[int]:
        """The tokens chosen by the step that ``launch`` gave ``ticket`` for (at most one newer step
        may have been launched since)."""
        if ticket < self.launched - 2:
            raise RuntimeError("the result of this decode step has been overwritten by later steps")
        self.result_event[ticket & 1].synchronize()
        # a bounded wait that ran out in one of the step's kernels: the tokens are not to be trusted
        kernels.raise_for_status(self.status_host[ticket & 1].tolist(), self.model.device)
        return self.result_host[ticket & 1][: self.live_of[ticket & 1]].tolist()

    def run(self, slots: list[int], tokens: list[int] | None, uniforms=None) -> list[int]:
        """One decode step for ``slots``, waited for."""
        return self.fetch(self.launch(slots, tokens, uniforms))


#: ``DRYFT_DECODE_PLACES=exact``: buffers of exactly the number of sequences (for measurements)
EXACT_PLACES = os.environ.get("DRYFT_DECODE_PLACES", "") == "exact"


def decode_places(n: int) -> int:
    """The size of the buffers that a decode step of ``n`` sequences runs on: ``n`` itself up to 8, then 16, 32
    and 64 (the sizes at which the decode products change their tile), beyond that the next multiple of 32.
    A large live set that loses its sequences one by one passes through few sizes, each of which costs a step
    launched kernel by kernel and a graph capture at its first two uses (about 40 ms at 36 layers); the places
    to spare cost 0 to 4 % of a step (measured at Qwen3-4B sizes: 9 sequences on 16 places at context 4,096
    3.15 against 3.02 ms, 24 on 32 4.57 against 4.47, 48 on 64 7.13 against 7.14).  Small batches keep their
    own size: three sequences on four places lost 6 % at context 4,096."""
    if EXACT_PLACES or n <= 8:
        return n
    if n <= 64:
        return 1 << (n - 1).bit_length()
    return -(-n // 32) * 32


class Decoder:
    """Keeps one ``DecodeBatch`` per size of buffers and remembers which slots ran last, so that a
    batch that goes on unchanged feeds its tokens back without a trip through the host."""

    def __init__(self, model, cache, use_graph: bool):
        self.model, self.cache = model, cache
        self.use_graph = use_graph and model.graph_safe
        self.batches: dict[tuple, DecodeBatch] = {}
        self.last: tuple | None = None

    def _batch_for(self, n: int, params: SamplingParams) -> tuple[tuple, DecodeBatch]:
        cache = self.cache
        widths = [max(1, -(-(g.ring_tokens or cache.max_context) // cache.page_size)) for g in cache.groups]
        places = decode_places(n)
        key = (places, tuple(widths), params.temperature)
        batch = self.batches.get(key)
        if batch is None:
            if len(self.batches) >= 32:
                self.batches.pop(next(iter(self.batches)))
            batch = self.batches[key] = DecodeBatch(self.model, cache, places, widths, cache.max_context,
                                                    params.temperature, self.use_graph)
        return key, batch

    def decode_launch(self, slots: list[int], tokens: list[int] | None, requests: list[int], step_index: int,
                      params: SamplingParams):
        """Starts one decode step and returns a handle whose ``result()`` gives the chosen tokens.
        ``tokens`` None: ``slots`` are the slots of the step launched last, fed what that step chose."""
        key, batch = self._batch_for(len(slots), params)
        if tokens is None and self.last != (key, tuple(slots)):
            raise ValueError("tokens=None needs the same slots as the decode step launched last")
        uniforms = None
        if params.temperature > 0:
            uniforms = [uniform_for(params.seed, r, step_index) for r in requests]
        ticket = batch.launch(list(slots), None if tokens is None else list(tokens), uniforms)
        self.last = (key, tuple(slots))
        return DecodeHandle(batch, ticket)

    def step_logits(self, slots: list[int], tokens: list[int]) -> torch.Tensor:
        """One decode step for ``slots`` fed ``tokens`` on the fixed buffers (and through the graph) that
        generation uses, waited for; returns the step's float32 logits ``[len(slots), vocab]``, which stay
        valid until the next step of this batch size.  The tokens the sampler chose are thrown away."""
        key, batch = self._batch_for(len(slots), SamplingParams())
        batch.fetch(batch.launch(list(slots), list(tokens)))
        self.last = None                  # the next decode step is fed from the host again
        batch.last_out = None
        return batch.logits[: len(slots)]

    def decode(self, slots: list[int], tokens: list[int], requests: list[int], step_index: int,
               params: SamplingParams) -> list[int]:
        key, batch = self._batch_for(len(slots), params)
        same = self.last == (key, tuple(slots)) and batch.last_out == list(tokens)
        out = self.decode_launch(slots, None if same else tokens, requests, step_index, params).result()
        batch.last_out = out
        return out


class DecodeHandle:
    """A decode step that has been launched; ``result()`` waits for it and returns its tokens."""

    def __init__(self, batch: DecodeBatch, ticket: int):
        self.batch, self.ticket = batch, ticket

    def result(self) -> list[int]:
        out = self.batch.fetch(self.ticket)
        self.batch.last_out = out
        return out
