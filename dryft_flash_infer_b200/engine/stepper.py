"""The step function: one batch of sequences, the tokens it is given, logits at the wanted places."""

from __future__ import annotations

import torch

from ..cache import SequenceCache
from .context import StepContext, StepEntry
from .prefill import PrefillGraphs


class Stepper:
    """Runs steps of a model over a cache.

    ``step(entries)`` takes, for each sequence, its slot and its next tokens: whole
    prompts of unequal lengths, one token each, or any mix.  It runs exactly these tokens
    as one packed batch, reading earlier tokens from the cache, appends their keys and
    values, advances each slot's length, and returns float32 logits ``[wanted, vocab]``
    in the order of the entries and of each entry's ``want`` (None if nothing is wanted).

    Groups of the cache that keep a window hold ``window + step_tokens - 1`` places per
    sequence, so a sequence's share of one pass is limited to ``step_tokens``; longer
    shares are cut into passes here, which changes no result.
    """

    def __init__(self, model, cache: SequenceCache, step_tokens: int, use_graph: bool = False, decoder=None):
        self.model, self.cache = model, cache
        self.step_tokens = step_tokens
        # with graphs on, a step of one token per sequence runs where generation's decode steps run: on
        # the decoder's fixed buffers, through its CUDA graph
        self.decoder = decoder if decoder is not None and decoder.use_graph else None
        # short prompt steps run as CUDA graphs at a few fixed shapes, if every mixer can be captured
        self.graphs = PrefillGraphs(model, cache) if use_graph and model.graph_safe else None
        self.has_ring = any(g.ring_tokens for g in cache.groups)
        self.device = model.device

    @torch.no_grad()
    def step(self, entries: list[StepEntry]):
        for e in entries:
            if len(e.tokens) == 0 and len(e.want) > 0:
                raise ValueError(f"wanted places {list(e.want)} of slot {e.slot}, which brings no tokens to this step")
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        vocab = self.model.spec.vocab_size
        for e in entries:
            for t in e.tokens:
                if not 0 <= t < vocab:
                    raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        longest = max(len(e.tokens) for e in entries)
        if longest == 1 and self.decoder is not None:
            return self._decode_pass(entries)
        if not self.has_ring or longest <= self.step_tokens:
            return self._pass(entries)
        # cut long shares into passes of at most step_tokens per sequence
        pieces, order = [], []
        for start in range(0, longest, self.step_tokens):
            batch = []
            for index, e in enumerate(entries):
                chunk = e.tokens[start:start + self.step_tokens]
                if not chunk:
                    continue
                want = []
                for place, w in enumerate(e.want):
                    if start <= w < start + len(chunk):
                        want.append(w - start)
                        order.append((index, place))
                batch.append(StepEntry(e.slot, chunk, want))
            out = self._pass(batch)
            if out is not None:
                pieces.append(out)
        if not pieces:
            return None
        logits = torch.cat(pieces)
        rank = sorted(range(len(order)), key=lambda i: order[i])
        return logits[torch.tensor(rank, device=logits.device)]

    def _decode_pass(self, entries: list[StepEntry]):
        for e in entries:
            if any(w != 0 for w in e.want):
                raise ValueError(f"wanted place {e.want} is outside the 1 token given for slot {e.slot}")
        logits = self.decoder.step_logits([e.slot for e in entries], [e.tokens[0] for e in entries])
        rows = [i for i, e in enumerate(entries) for _ in e.want]
        if not rows:
            return None
        if rows == list(range(len(entries))):
            return logits.clone()
        return logits[torch.tensor(rows, device=logits.device)]

    def _pass(self, entries: list[StepEntry]):
        for e in entries:
            self.cache.book.reserve(e.slot, len(e.tokens))
        logits = self.graphs.run(entries) if self.graphs is not None else None
        if logits is None:
            ctx = StepContext(entries, self.cache, self.device)
            logits = self.model.forward(ctx, self.cache)
        for e in entries:
            self.cache.book.advance(e.slot, len(e.tokens))
        return logits
