"""The programming entry point: ``Engine(model_path).generate(input_ids, max_new_tokens)``.

The class keeps the shape of the reference's contract (engine/engine.py:179-217,
:1121-1157; README.md:54-66): built from a model folder, ``generate`` is a generator that
yields one list with one token per sequence for each output step.  What the
reference sets through ``DRYFT_*`` environment variables (engine/engine.py:45-155) are
keyword arguments here.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache import PAGE_SIZE, SequenceCache
from ..config import ModelConfig, architecture_named, config_from_dict, load_config
from ..ops import kernels
from ..sampling import SamplingParams, select_tokens
from ..weights import fill_random, load_weights
from .context import StepEntry
from .decode import Decoder
from .generate import Request, generate_all, generate_batch
from .model import DecoderModel
from .stepper import Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def _round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


@dataclass
class EngineOptions:
    """``dtype``: ``bfloat16`` runs the serving kernels, ``float32`` the whole model in true
    32-bit.  ``max_tokens``: token places that live sequences may hold together, each
    sequence rounded up to a page of 64; with ``max_seqs`` and ``max_context`` it sizes the
    cache once.  Left at None the cache is sized (and re-sized between batches) by what
    ``generate`` is asked for.  ``step_tokens``: the share of one pass per sequence in
    cache groups that keep a window."""

    dtype: str = "bfloat16"
    max_tokens: int | None = None
    max_seqs: int | None = None
    max_context: int | None = None
    step_tokens: int = 512
    #: capture the decode step in a CUDA graph; the default follows the reference's
    #: DRYFT_GRAPH=on|off environment variable (engine/engine.py:79)
    cuda_graph: bool = os.environ.get("DRYFT_GRAPH", "on") == "on"
    device: str = "cuda:0"


class Engine:
    def __init__(self, model_path: str | Path | None = None, *, config: ModelConfig | dict | None = None,
                 random_weights: bool = False, seed: int = 0, **options):
        self.options = EngineOptions(**options)
        if self.options.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {self.options.dtype!r}")
        self.dtype = _DTYPES[self.options.dtype]
        if not torch.cuda.is_available():
            raise RuntimeError("dryft-flash-infer_b200 runs on a CUDA device (sm_100a) only: none is visible, "
                               "and there is no CPU path")
        self.device = torch.device(self.options.device)
        torch.cuda.set_device(self.device)
        # true float32 products: no reduced-precision matrix mode anywhere (engine/engine.py:182-183)
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")

        if model_path is not None:
            if config is not None or random_weights:
                raise ValueError("give either a model folder, or a configuration with random_weights=True")
            self.config = load_config(model_path)
        else:
            if config is None or not random_weights:
                raise ValueError("without a model folder, give config=... and random_weights=True")
            self.config = config_from_dict(config) if isinstance(config, dict) else config
        spec = architecture_named(self.config.architecture).build(self.config)
        self.model = DecoderModel(spec)
        self.model.allocate(self.dtype, self.device)
        if model_path is not None:
            load_weights(self.model, model_path)
        else:
            fill_random(self.model, seed)

        self.cache: SequenceCache | None = None
        self.stepper: Stepper | None = None
        self.decoder: Decoder | None = None
        self._positions_ready = 0
        if self.options.max_tokens is not None:
            max_tokens = _round_up(self.options.max_tokens, PAGE_SIZE)
            max_seqs = self.options.max_seqs or max(1, max_tokens // PAGE_SIZE)
            max_context = self.options.max_context or min(max_tokens, spec.max_positions)
            self._make_cache(max_tokens, max_seqs, max_context)

    # ------------------------------------------------------------------ cache
    def _make_cache(self, max_tokens: int, max_seqs: int, max_context: int) -> None:
        if max_context > self.model.spec.max_positions:
            raise ValueError(f"max_context {max_context} exceeds the model's max_position_embeddings "
                             f"{self.model.spec.max_positions}")
        self.cache = self.stepper = self.decoder = None
        torch.cuda.empty_cache()
        kv_needs, state_needs = self.model.cache_needs()
        self.cache = SequenceCache(kv_needs, state_needs, max_tokens=max_tokens, max_seqs=max_seqs,
                                   max_context=max_context, step_tokens=self.options.step_tokens,
                                   dtype=self.dtype, device=self.device)
        if max_context > self._positions_ready:
            self.model.prepare(max_context)
            self._positions_ready = max_context
        self.decoder = Decoder(self.model, self.cache, self.options.cuda_graph)
        self.stepper = Stepper(self.model, self.cache, self.options.step_tokens, self.options.cuda_graph, self.decoder)

    def _ensure_room(self, lengths: list[int]) -> None:
        """Makes the cache fit a batch whose sequences reach ``lengths`` tokens."""
        need_tokens = sum(_round_up(n, PAGE_SIZE) for n in lengths)
        need_context = max(lengths)
        c = self.cache
        if c is not None:
            free_tokens = min(g.pages.pool.free for g in c.groups if not g.ring_tokens) * PAGE_SIZE \
                if any(not g.ring_tokens for g in c.groups) else need_tokens
            if (free_tokens >= need_tokens and c.book.slots.free >= len(lengths)
                    and c.max_context >= need_context):
                return
            if self.options.max_tokens is not None or c.live_slots:
                raise RuntimeError(
                    f"the cache (max_tokens={c.max_tokens}, max_seqs={c.max_seqs}, max_context={c.max_context}) "
                    f"cannot take a batch of {len(lengths)} sequences needing {need_tokens} token places")
        self._make_cache(need_tokens, len(lengths), _round_up(need_context, PAGE_SIZE))

    # ------------------------------------------------------------------ backend of the generation loop
    def open_slot(self) -> int:
        return self.cache.open_slot()

    def close_slot(self, slot: int) -> None:
        self.cache.close_slot(slot)

    def step(self, entries: list[StepEntry]):
        """See ``Stepper.step``."""
        if self.stepper is None:
            raise RuntimeError("the engine has no cache yet: build it with max_tokens=..., or call generate")
        return self.stepper.step(entries)

    def decode(self, slots: list[int], tokens: list[int], requests: list[int], step_index: int,
               params: SamplingParams) -> list[int]:
        """One decode step for ``slots`` fed ``tokens``; returns the tokens chosen next.  The
        step runs on fixed buffers (as a CUDA graph unless switched off) and samples on the
        device, so no logits cross to the host."""
        return self.decoder.decode(slots, tokens, requests, step_index, params)

    def decode_launch(self, slots: list[int], tokens: list[int] | None, requests: list[int], step_index: int,
                      params: SamplingParams):
        """Like ``decode`` without the wait: returns a handle whose ``result()`` gives the tokens.  With
        ``tokens`` None the step is fed what the step launched last chose, which never left the device."""
        return self.decoder.decode_launch(slots, tokens, requests, step_index, params)

    def select(self, logits, requests: list[int], step_index: int, params: SamplingParams) -> list[int]:
        chosen = select_tokens(logits, params, requests, step_index).tolist()
        self.check_status()               # the tokens are on the host: so is anything the step's kernels recorded
        return chosen

    def check_status(self) -> None:
        """Raises ``KernelError`` if a bounded wait ran out in a kernel launched since the last check (the
        results computed since are then not valid).  It synchronises; ``select`` and the decode steps'
        ``result()`` check for themselves, a caller of ``step`` alone calls it once its logits are on the host."""
        kernels.check_status(self.device)

    # ------------------------------------------------------------------ generation
    def generate(self, input_ids: list[list[int]], max_new_tokens: int, *, temperature: float = 0.0, seed: int = 0,
                 stop_token_ids: tuple[int, ...] = ()) -> Iterator[list[int | None]]:
        """Continues every sequence of ``input_ids`` (prompts may differ in length).

        Yields, for each output step, a list with one token id per sequence, exactly
        ``max_new_tokens`` times when no stop tokens are given (the default, and the
        reference's behaviour).  With ``stop_token_ids`` a sequence ends with its first
        stop token and shows as None afterwards.  ``temperature`` 0 is greedy.
        """
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must be nonnegative")
        if max_new_tokens == 0 or not input_ids:
            return
        requests = [Request(list(map(int, p)), max_new_tokens, tuple(stop_token_ids), request_id=i)
                    for i, p in enumerate(input_ids)]
        self._ensure_room([len(r.prompt) + max_new_tokens for r in requests])
        yield from generate_batch(self, requests, SamplingParams(temperature, seed))

    def generate_requests(self, requests: list[Request], *, max_batch: int = 64, temperature: float = 0.0,
                          seed: int = 0) -> list[Request]:
        """Runs any number of requests, ``max_batch`` at a time, one batch after another;
        each request's tokens end up in its ``output``."""
        if not requests:
            return []
        longest = sorted((len(r.prompt) + r.max_new_tokens for r in requests), reverse=True)[:max_batch]
        self._ensure_room(longest)
        return generate_all(self, requests, SamplingParams(temperature, seed), max_batch)
