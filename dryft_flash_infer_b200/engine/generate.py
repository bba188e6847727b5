"""The generation loop: batches of prompts in, tokens out, step by step.

The loop only decides: which sequences run in a step, what they are given, when one
ends and gives its slot back, when a batch ends and the next one starts.  The work is
done by a *backend* with four methods, so that the decisions can be tested without a
device:

    open_slot() -> slot            close_slot(slot)
    step(entries) -> logits        (entries: list of StepEntry; one logits row per wanted place)
    select(logits, requests, step_index, params) -> list[int]
    decode(slots, tokens, requests, step_index, params) -> list[int]     (optional)
    decode_launch(slots, tokens or None, requests, step_index, params) -> handle with result()   (optional)

``decode`` is one step of one token per sequence with the choice of the next token
folded in; a backend that has it is given the decode steps whole, so that it can keep
them on the device.  With ``decode_launch`` the loop starts the next step before it reads
the tokens of the one before (as the reference's stream stays one step ahead of the host,
engine/engine.py:1159-1185) whenever it knows without them who goes on: no stop tokens, and
nobody reaches its length at this step.

Behaviour follows the reference's ``generate`` (engine/engine.py:1121-1157): one list
with one token per sequence for every output step, exactly ``max_new_tokens`` of them,
the last token never fed back; a negative count is an error and zero does no work.
Added to it: prompts of unequal lengths, and stop tokens.  A sequence that ends early
(its stop token is the last one it yields) gives its slot back at once and shows as
``None`` in later lists; the batch ends when all its sequences have ended.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Iterator

from ..sampling import SamplingParams
from .context import StepEntry


@dataclass
class Request:
    """One prompt and its limits; ``output`` collects what is generated for it."""

    prompt: list[int]
    max_new_tokens: int
    stop_token_ids: tuple[int, ...] = ()
    request_id: int = 0
    output: list[int] = field(default_factory=list)
    finish_reason: str | None = None


def generate_batch(backend, requests: list[Request], params: SamplingParams) -> Iterator[list[int | None]]:
    """Runs ``requests`` as one batch that starts together; yields one list per output step."""
    for r in requests:
        if r.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be nonnegative")
        if not r.prompt:
            raise ValueError("a prompt needs at least one token")
    live = [i for i, r in enumerate(requests) if r.max_new_tokens > 0]
    if not live:
        return
    slots: dict[int, int] = {}
    try:
        for i in live:
            slots[i] = backend.open_slot()
        # all prompts in one step; only each prompt's last place is wanted
        entries = [StepEntry(slots[i], list(requests[i].prompt), [len(requests[i].prompt) - 1]) for i in live]
        step_index = 0
        fused_decode = getattr(backend, "decode", None)
        launch_decode = getattr(backend, "decode_launch", None)
        if any(requests[i].stop_token_ids for i in live):
            launch_decode = None                      # who goes on depends on the tokens themselves
        in_flight = None                              # a launched step whose tokens have not been read
        while live:
            ids = [requests[i].request_id for i in live]
            ahead = None
            if step_index == 0:
                chosen = backend.select(backend.step(entries), ids, step_index, params)
            elif launch_decode is not None:
                if in_flight is None:
                    in_flight = launch_decode([slots[i] for i in live], [requests[i].output[-1] for i in live], ids,
                                              step_index, params)
                # if nobody ends with the step in flight, the one after it can start before its tokens are read
                if all(len(requests[i].output) + 1 < requests[i].max_new_tokens for i in live):
                    ahead = launch_decode([slots[i] for i in live], None, ids, step_index + 1, params)
                chosen = in_flight.result()
            elif fused_decode is not None:
                chosen = fused_decode([slots[i] for i in live], [requests[i].output[-1] for i in live], ids,
                                      step_index, params)
            else:
                chosen = backend.select(backend.step(entries), ids, step_index, params)
            in_flight = ahead
            row: list[int | None] = [None] * len(requests)
            still = []
            for i, token in zip(live, chosen):
                r = requests[i]
                token = int(token)
                r.output.append(token)
                row[i] = token
                if token in r.stop_token_ids:
                    r.finish_reason = "stop"
                elif len(r.output) >= r.max_new_tokens:
                    r.finish_reason = "length"
                if r.finish_reason is None:
                    still.append(i)
                else:
                    backend.close_slot(slots.pop(i))
            yield row
            live = still
            entries = [StepEntry(slots[i], [requests[i].output[-1]], [0]) for i in live]
            step_index += 1
    finally:
        # a generator closed early, or an error: nothing stays held
        for slot in slots.values():
            backend.close_slot(slot)
        slots.clear()


def generate_all(backend, requests: Iterable[Request], params: SamplingParams, max_batch: int,
                 batch_token_budget: int | None = None) -> list[Request]:
    """Runs any number of requests, ``max_batch`` at a time, one batch after another.

    A batch is cut earlier if its prompts and outputs together would need more than
    ``batch_token_budget`` token places (each sequence rounded up by the caller's unit).
    """
    pending = list(requests)
    done: list[Request] = []
    while pending:
        batch, need = [], 0
        while pending and len(batch) < max_batch:
            r = pending[0]
            cost = len(r.prompt) + r.max_new_tokens
            if batch_token_budget is not None and batch and need + cost > batch_token_budget:
                break
            batch.append(pending.pop(0))
            need += cost
        for _ in generate_batch(backend, batch, params):
            pass
        done.extend(batch)
    return done
