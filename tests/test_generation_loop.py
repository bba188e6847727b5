"""The generation loop's decisions, with a backend that needs no device."""

import pytest

from dryft_flash_infer_b200.engine.generate import Request, generate_all, generate_batch
from dryft_flash_infer_b200.sampling import SamplingParams, uniform_for


class FakeBackend:
    """Next token = (sum of the sequence so far) % 50; records what it is asked to do."""

    def __init__(self, n_slots=8):
        self.free = list(range(n_slots))
        self.held = {}          # slot -> tokens seen so far
        self.steps = []         # per step: list of (slot, n_tokens)
        self.opened = []
        self.closed = []

    def open_slot(self):
        slot = self.free.pop(0)
        self.held[slot] = []
        self.opened.append(slot)
        return slot

    def close_slot(self, slot):
        assert slot in self.held, "slot freed twice"
        del self.held[slot]
        self.free.insert(0, slot)
        self.closed.append(slot)

    def step(self, entries):
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            assert e.slot in self.held
            self.held[e.slot].extend(e.tokens)
            assert e.want == [len(e.tokens) - 1]
            rows.append(sum(self.held[e.slot]) % 50)
        return rows

    def select(self, logits, requests, step_index, params):
        self.last_requests = list(requests)
        return list(logits)


def expected(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(sum(seq) % 50)
        seq.append(out[-1])
    return out


def test_unequal_prompts_in_one_prefill_then_one_token_each():
    backend = FakeBackend()
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    requests = [Request(p, 4, request_id=i) for i, p in enumerate(prompts)]
    rows = list(generate_batch(backend, requests, SamplingParams()))
    assert len(rows) == 4 and all(len(r) == 3 for r in rows)
    for i, p in enumerate(prompts):
        assert [r[i] for r in rows] == expected(p, 4) == requests[i].output
    assert [n for _, n in backend.steps[0]] == [3, 1, 5]                 # all prompts in the first step
    assert all(n == 1 for step in backend.steps[1:] for _, n in step)    # then one token each
    assert len(backend.steps) == 4                                       # the last token is not fed back
    assert backend.held == {} and sorted(backend.closed) == sorted(backend.opened)
    assert all(r.finish_reason == "length" for r in requests)


def test_stop_token_ends_a_sequence_early_and_frees_its_slot():
    backend = FakeBackend()
    prompts = [[1, 2, 3], [10, 20]]
    stop = expected(prompts[0], 2)[1]
    requests = [Request(p, 6, stop_token_ids=(stop,), request_id=i) for i, p in enumerate(prompts)]
    rows = list(generate_batch(backend, requests, SamplingParams()))
    first = expected(prompts[0], 6)
    cut = first.index(stop) + 1
    assert requests[0].output == first[:cut] and requests[0].finish_reason == "stop"
    assert [r[0] for r in rows[cut:]] == [None] * (len(rows) - cut)
    assert requests[1].output == expected(prompts[1], 6) or requests[1].finish_reason == "stop"
    # after the early end, steps carry one sequence only
    assert all(len(step) == 1 for step in backend.steps[cut:])
    assert backend.held == {}


def test_different_lengths_and_zero_and_negative():
    backend = FakeBackend()
    requests = [Request([1], 1), Request([2], 3), Request([3], 0)]
    rows = list(generate_batch(backend, requests, SamplingParams()))
    assert len(rows) == 3 and rows[0][2] is None and rows[1][0] is None
    assert requests[2].output == [] and len(backend.opened) == 2
    assert list(generate_batch(backend, [Request([1], 0)], SamplingParams())) == [] and len(backend.steps) == 3
    with pytest.raises(ValueError):
        list(generate_batch(backend, [Request([1], -1)], SamplingParams()))
    with pytest.raises(ValueError):
        list(generate_batch(backend, [Request([], 2)], SamplingParams()))


def test_closing_the_generator_early_gives_everything_back():
    backend = FakeBackend()
    gen = generate_batch(backend, [Request([1, 2], 10), Request([3], 10)], SamplingParams())
    next(gen)
    next(gen)
    gen.close()
    assert backend.held == {} and sorted(backend.closed) == sorted(backend.opened)


def test_an_error_in_a_step_gives_everything_back():
    backend = FakeBackend()
    original = backend.step

    def failing(entries):
        if len(backend.steps) == 2:
            raise RuntimeError("boom")
        return original(entries)

    backend.step = failing
    with pytest.raises(RuntimeError):
        list(generate_batch(backend, [Request([1, 2], 10), Request([3], 10)], SamplingParams()))
    assert backend.held == {}


def test_many_requests_run_batch_after_batch_and_reuse_slots():
    backend = FakeBackend(n_slots=3)
    prompts = [[i + 1, i + 2] for i in range(8)]
    requests = [Request(p, 2 + i % 3, request_id=i) for i, p in enumerate(prompts)]
    done = generate_all(backend, requests, SamplingParams(), max_batch=3)
    assert [r.output for r in done] == [expected(p, 2 + i % 3) for i, p in enumerate(prompts)]
    assert len(backend.opened) == 8 and set(backend.opened) == {0, 1, 2}   # three slots serve eight requests
    assert backend.held == {}
    # a token budget cuts batches earlier
    backend = FakeBackend()
    requests = [Request([1] * 10, 5, request_id=i) for i in range(4)]
    generate_all(backend, requests, SamplingParams(), max_batch=4, batch_token_budget=30)
    assert [len(s) for s in backend.steps if s and s[0][1] == 10] == [2, 2]


def test_request_ids_reach_the_sampler_and_uniforms_do_not_depend_on_the_batch():
    backend = FakeBackend()
    list(generate_batch(backend, [Request([1], 1, request_id=41), Request([2], 1, request_id=7)], SamplingParams(0.8, 3)))
    assert backend.last_requests == [41, 7]
    u = uniform_for(3, 41, 5)
    assert 0.0 <= u < 1.0 and u == uniform_for(3, 41, 5)
    assert len({uniform_for(3, r, s) for r in range(20) for s in range(20)}) > 390
    assert abs(sum(uniform_for(1, r, 0) for r in range(4000)) / 4000 - 0.5) < 0.03


class AsyncBackend(FakeBackend):
    """A backend that can start a decode step without waiting for it; it logs what happens in order."""

    def __init__(self):
        super().__init__()
        self.log = []
        self.device_tokens = {}

    def decode_launch(self, slots, tokens, requests, step_index, params):
        backend = self
        if tokens is None:                       # fed from the device: what the step launched last chose
            tokens = [backend.device_tokens[s] for s in slots]
            self.log.append(("launch-from-device", step_index))
        else:
            self.log.append(("launch-from-host", step_index))
        chosen = []
        for slot, token in zip(slots, tokens):
            self.held[slot].append(token)
            chosen.append(sum(self.held[slot]) % 50)
            backend.device_tokens[slot] = chosen[-1]

        class Handle:
            def result(self_inner):
                backend.log.append(("read", step_index))
                return chosen

        return Handle()


def test_the_next_step_starts_before_the_last_one_is_read():
    backend = AsyncBackend()
    prompts = [[1, 2, 3], [4, 5]]
    requests = [Request(p, 5, request_id=i) for i, p in enumerate(prompts)]
    rows = list(generate_batch(backend, requests, SamplingParams()))
    assert [[r[i] for r in rows] for i in range(2)] == [expected(p, 5) for p in prompts]
    # step 1 is launched with host tokens, steps 2.. from the device, each before the step before it is read;
    # the last step (4) is not followed by another launch
    assert backend.log == [("launch-from-host", 1), ("launch-from-device", 2), ("read", 1), ("launch-from-device", 3),
                           ("read", 2), ("launch-from-device", 4), ("read", 3), ("read", 4)]
    assert backend.held == {}


def test_lookahead_stops_where_a_sequence_ends_and_with_stop_tokens():
    backend = AsyncBackend()
    requests = [Request([1, 2, 3], 3, request_id=0), Request([4, 5], 5, request_id=1)]
    rows = list(generate_batch(backend, requests, SamplingParams()))
    assert requests[0].output == expected([1, 2, 3], 3) and requests[1].output == expected([4, 5], 5)
    assert rows[3][0] is None and rows[4][0] is None
    # step 2 ends request 0: nothing is launched ahead of it; step 3 starts from the host with the survivor
    assert ("launch-from-host", 3) in backend.log and ("launch-from-device", 3) not in backend.log
    assert backend.log.index(("read", 2)) < backend.log.index(("launch-from-host", 3))
    # with stop tokens nothing is ever launched ahead
    backend = AsyncBackend()
    backend.decode = lambda slots, tokens, requests, step_index, params: \
        backend.decode_launch(slots, tokens, requests, step_index, params).result()
    list(generate_batch(backend, [Request([1, 2, 3], 4, stop_token_ids=(49,))], SamplingParams()))
    assert all(kind != "launch-from-device" for kind, _ in backend.log)


def test_sizes_of_decode_buffers_and_hints_without_a_gpu():
    """Decisions that need no device: which size of buffers a live set of n sequences decodes on, and that a
    hint about the next weights is nothing where the decode kernels would not run (and keeps no matrix alive)."""
    import gc

    import torch

    from dryft_flash_infer_b200.engine.decode import decode_places
    from dryft_flash_infer_b200.ops import kernels

    sizes = [decode_places(n) for n in range(1, 130)]
    assert sizes[:8] == list(range(1, 9))                                    # small batches keep their own size
    assert all(a <= b for a, b in zip(sizes, sizes[1:]))                      # never fewer places for more sequences
    assert all(size >= n for n, size in enumerate(sizes, start=1))
    assert sorted(set(sizes[8:64])) == [16, 32, 64]                           # the sizes at which the products change their tile
    assert sorted(set(sizes[64:])) == [96, 128, 160]                          # beyond 64: multiples of 32
    assert all(size - n < max(32, n) for n, size in enumerate(sizes, start=1))    # never more filling than sequences (or 32 places)

    # what a decode step says about how long its sequences may get: the smallest limit that covers the longest,
    # never more than the cache's own, never less than the longest
    steps = kernels.DECODE_KV_STEPS
    assert list(steps) == sorted(steps)
    for max_context in (64, 2048, 4096, 6000, 40960):
        limits = [kernels.decode_kv_limit(n, max_context) for n in range(1, max_context + 1, 61)]
        assert all(a <= b for a, b in zip(limits, limits[1:])) and limits[-1] <= max_context
        assert all(limit >= n for limit, n in zip(limits, range(1, max_context + 1, 61)))
        assert set(limits) <= set(steps) | {max_context}
    assert kernels.decode_kv_limit(1, 40960) == steps[0] and kernels.decode_kv_limit(steps[0] + 1, 40960) == steps[1]
    assert kernels.decode_kv_limit(steps[-1] + 1, 40960) == 40960

    weight = torch.zeros(16, 32, dtype=torch.bfloat16)
    hint = kernels.next_weights(weight, swiglu=True)
    assert hint is kernels.next_weights(weight, swiglu=True) and hint is not kernels.next_weights(weight)
    assert hint.hint(8) is None                     # not on a device: the decode kernels would not run there
    assert kernels.next_weights(None) is None
    held = len(kernels._NEXT_WEIGHTS)
    del weight
    gc.collect()
    assert hint.weight is None and len(kernels._NEXT_WEIGHTS) == held - 2
