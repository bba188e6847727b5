"""What a step's kernels need to know about its rows, gathered once and uploaded in one copy."""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens (0-based) whose logits are wanted."""

    slot: int
    tokens: list[int]
    want: list[int] = field(default_factory=list)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class StepContext:
    """Rows of one step, packed sequence after sequence without padding.

    Device tensors (all int32): ``tokens [rows]``, ``row_seq [rows]`` (which sequence of
    the step a row belongs to), ``row_pos [rows]`` (its absolute position), ``seq_start``,
    ``seq_qlen``, ``seq_slot [seqs]``, ``cu_rows [seqs+1]``, ``wanted_rows [wanted]`` and
    one block table ``[seqs, width]`` per cache group.  Host copies of the per-sequence
    numbers stay in ``starts``, ``q_lens``, ``slots``.

    With ``shape = (rows, sequences, wanted)`` the step is laid out at these sizes, which are
    larger than its own, so that steps of different sizes share one set of buffers and one
    CUDA graph: the rows past the step's own belong to no sequence (``cu_rows`` ends before
    them), carry token 0 at position 0 of a last, empty sequence whose block table names the
    null page only, and so reach neither a live page nor another row; the wanted places
    past the step's own name row 0.  ``into`` is the fixed device buffer to upload into.
    """

    def __init__(self, entries: list[StepEntry], cache, device, table_widths: list[int] | None = None,
                 shape: tuple[int, int, int] | None = None, into: torch.Tensor | None = None):
        #: ``kernels.NextWeights`` of the matrix that the step streams after the part that is running, or
        #: None: the model and the blocks keep it up to date, a part may give it to its last kernel
        self.upcoming = None
        self.decode_plans = None          # set by the model for the length of one pass (see kernels.attention_decode)
        self.slots = [e.slot for e in entries]
        self.q_lens = [len(e.tokens) for e in entries]
        self.starts = [cache.length(e.slot) for e in entries]
        own_seqs = len(entries)
        own_rows = sum(self.q_lens)
        self.max_q_len = max(self.q_lens, default=0)
        self.max_kv_len = max((s + q for s, q in zip(self.starts, self.q_lens)), default=0)
        self.all_decode = all(q == 1 for q in self.q_lens)

        wanted = []
        base = 0
        for e, q in zip(entries, self.q_lens):
            for w in e.want:
                if not 0 <= w < q:
                    raise ValueError(f"wanted place {w} is outside the {q} tokens given for slot {e.slot}")
                wanted.append(base + w)
            base += q
        own_wanted = len(wanted)
        if shape is None:
            rows, n = own_rows, own_seqs
            self.wants_every_row = wanted == list(range(rows))
        else:
            rows, n, padded_wanted = shape
            if rows < own_rows or n <= own_seqs or padded_wanted < own_wanted:
                raise ValueError(f"a step of {own_rows} rows, {own_seqs} sequences and {own_wanted} wanted places does "
                                 f"not fit the shape {shape} (which needs one sequence to spare)")
            wanted = wanted + [0] * (padded_wanted - own_wanted)
            self.wants_every_row = False
            self.all_decode = False
            self.max_q_len = rows
            self.max_kv_len = cache.max_context
        self.n_seqs, self.n_rows, self.n_wanted = n, rows, len(wanted)
        self.own_rows, self.own_seqs, self.own_wanted = own_rows, own_seqs, own_wanted

        n_groups = len(cache.groups)
        if table_widths is None:
            table_widths = [cache.table_width(self.slots, g) for g in range(n_groups)]
        self.table_widths = table_widths

        # one int32 buffer, every section starting on a 16-byte boundary
        sections = {"tokens": rows, "row_seq": rows, "row_pos": rows, "seq_start": n, "seq_qlen": n,
                    "seq_slot": n, "cu_rows": n + 1, "wanted_rows": max(1, len(wanted))}
        for g in range(n_groups):
            sections[f"table{g}"] = n * table_widths[g]
        offsets, total = {}, 0
        for name, size in sections.items():
            offsets[name] = total
            total += _pad4(size)
        host = np.zeros(max(total, 4), dtype=np.int32)

        def view(name, size):
            return host[offsets[name]: offsets[name] + size]

        cu = np.full(n + 1, own_rows, dtype=np.int64)
        cu[0] = 0
        np.cumsum(self.q_lens, out=cu[1:own_seqs + 1])
        view("cu_rows", n + 1)[:] = cu
        tokens, row_seq, row_pos = view("tokens", rows), view("row_seq", rows), view("row_pos", rows)
        row_seq[own_rows:] = n - 1          # rows past the step's own: the empty sequence at the end
        for i, e in enumerate(entries):
            a, b = int(cu[i]), int(cu[i + 1])
            tokens[a:b] = e.tokens
            row_seq[a:b] = i
            row_pos[a:b] = np.arange(self.starts[i], self.starts[i] + (b - a))
        view("seq_start", own_seqs)[:] = self.starts
        view("seq_qlen", own_seqs)[:] = self.q_lens
        view("seq_slot", own_seqs)[:] = self.slots
        view("wanted_rows", len(wanted))[:] = wanted
        for g in range(n_groups):
            cache.fill_block_table(view(f"table{g}", n * table_widths[g]).reshape(n, table_widths[g])[:own_seqs],
                                   self.slots, g, table_widths[g])
        self.host = host
        self.offsets, self.sections = offsets, sections
        self.device_buffer = None
        self.upload(device, into)

    def upload(self, device, into: torch.Tensor | None = None) -> None:
        """Copies the packed numbers to the device (into a fixed buffer if one is given)."""
        staged = torch.from_numpy(self.host)
        if into is None:
            self.device_buffer = staged.to(device, non_blocking=False)
        else:
            into[: staged.numel()].copy_(staged, non_blocking=False)
            self.device_buffer = into
        buf = self.device_buffer

        def view(name, size):
            return buf[self.offsets[name]: self.offsets[name] + size]

        rows, n = self.n_rows, self.n_seqs
        self.tokens, self.row_seq, self.row_pos = view("tokens", rows), view("row_seq", rows), view("row_pos", rows)
        self.seq_start, self.seq_qlen, self.seq_slot = view("seq_start", n), view("seq_qlen", n), view("seq_slot", n)
        self.cu_rows = view("cu_rows", n + 1)
        self.wanted_rows = view("wanted_rows", self.n_wanted)
        self.block_tables = [view(f"table{g}", n * w).view(n, w) for g, w in enumerate(self.table_widths)]
