"""A decoder assembled from a ``ModelSpec``: parts, weights and the forward pass of a step."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels
from ..parts import ModelSpec, Part, TensorDecl, build_part, part_factory


@dataclass(frozen=True)
class ExpectedTensor:
    """A tensor of the model file and where it goes: ``owner`` is the part (or the model
    itself for embedding and head), ``decl`` says which rows of which buffer."""

    name: str
    decl: TensorDecl
    owner: object


class DecoderModel:
    """Embedding, the scheduled blocks, the final norm and the output head.

    Built from the spec alone; ``allocate`` makes the device buffers and ``bind`` hands
    them to the parts once a loader has filled them.  ``forward`` runs the rows of one
    step through the schedule and returns float32 logits for the wanted rows.
    """

    def __init__(self, spec: ModelSpec):
        spec.check()
        self.spec = spec
        self.blocks = []
        for layer in spec.layers:
            block_class = part_factory("block", layer.block)
            self.blocks.append(block_class(
                build_part("mixer", layer.mixer, spec.hidden_size),
                build_part("feed_forward", layer.feed_forward, spec.hidden_size),
                {name: build_part("norm", norm, spec.hidden_size) for name, norm in layer.norms.items()}))
        self.final_norm = build_part("norm", spec.final_norm, spec.hidden_size) if spec.final_norm is not None else None
        self.embedding = None   # [vocab, hidden]
        self.head = None        # [vocab, hidden]; the embedding itself when tied
        self.dtype = None
        self.device = None
        self._buffers: dict[int, dict[str, torch.Tensor]] = {}

    # ------------------------------------------------------------------ tensors
    def expected_tensors(self) -> list[ExpectedTensor]:
        spec = self.spec
        out = [ExpectedTensor(spec.embedding_name,
                              TensorDecl((spec.vocab_size, spec.hidden_size), "embedding"), self)]
        for layer, block in zip(spec.layers, self.blocks):
            for part_name, part in block.parts().items():
                for local, decl in part.tensors().items():
                    key = f"{part_name}.{local}"
                    if key not in layer.tensor_names:
                        raise ValueError(f"the architecture gives no file name for tensor '{key}'")
                    out.append(ExpectedTensor(layer.tensor_names[key], decl, part))
        if self.final_norm is not None:
            for local, decl in self.final_norm.tensors().items():
                out.append(ExpectedTensor(spec.final_norm_names[local], decl, self.final_norm))
        if spec.head_name is not None:
            out.append(ExpectedTensor(spec.head_name, TensorDecl((spec.vocab_size, spec.hidden_size), "head"), self))
        names = [t.name for t in out]
        if len(set(names)) != len(names):
            raise ValueError("the architecture names a file tensor twice")
        return out

    def _parts(self) -> list[Part]:
        parts: list[Part] = []
        for block in self.blocks:
            parts.extend(block.parts().values())
        if self.final_norm is not None:
            parts.append(self.final_norm)
        return parts

    @property
    def graph_safe(self) -> bool:
        """True if every part says that a decode step through it can be captured in a CUDA graph."""
        return all(part.graph_safe for part in self._parts())

    def allocate(self, dtype: torch.dtype, device) -> None:
        """Creates every part's device buffers (uninitialised)."""
        self.dtype, self.device = dtype, device
        for part in self._parts():
            held = {}
            for name, (shape, precision) in part.buffer_shapes().items():
                held[name] = torch.empty(shape, dtype=dtype if precision == "compute" else torch.float32,
                                         device=device)
            self._buffers[id(part)] = held
        own = {"embedding": torch.empty((self.spec.vocab_size, self.spec.hidden_size), dtype=dtype, device=device)}
        if self.spec.head_name is not None:
            own["head"] = torch.empty((self.spec.vocab_size, self.spec.hidden_size), dtype=dtype, device=device)
        self._buffers[id(self)] = own

    def destination(self, expected: ExpectedTensor) -> torch.Tensor:
        """The rows of a device buffer that ``expected`` fills."""
        buffer = self._buffers[id(expected.owner)][expected.decl.buffer]
        return buffer[expected.decl.row_start: expected.decl.row_start + expected.decl.shape[0]]

    def bind(self) -> None:
        for part in self._parts():
            part.bind(self._buffers[id(part)])
        own = self._buffers[id(self)]
        self.embedding = own["embedding"]
        self.head = own.get("head", self.embedding)

    def prepare(self, max_positions: int) -> None:
        for block in self.blocks:
            block.mixer.prepare(max_positions, self.device)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for held in self._buffers.values():
            for t in held.values():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self):
        """``({cache id: KVNeed}, {schedule position: StateNeed})`` over the schedule."""
        kv, state = {}, {}
        for position, entry in enumerate(self.spec.schedule):
            mixer = self.blocks[entry.layer].mixer
            need = mixer.cache_need()
            if need is not None:
                if entry.cache in kv and kv[entry.cache] != need:
                    raise ValueError(f"schedule[{position}] shares cache {entry.cache} with a layer of another shape")
                kv[entry.cache] = need
            wanted = mixer.state_need()
            if wanted is not None:
                state[position] = wanted
        return kv, state

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, cache) -> torch.Tensor | None:
        """Runs ``ctx``'s rows through the model; logits float32 ``[wanted rows, vocab]``."""
        with kernels.on_current_stream():
            return self._forward(ctx, cache)

    def _forward(self, ctx, cache) -> torch.Tensor | None:
        spec = self.spec
        ctx.decode_plans = {}       # what the kernels of this pass work out once and share between layers
        residual = kernels.embedding(self.embedding, ctx.tokens, scale=spec.embedding_scale)
        pending = None
        schedule = self.spec.schedule
        for position, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            view = cache.layer_view(entry.cache, ctx.block_tables, entry.writes_cache) \
                if block.mixer.cache_need() is not None else None
            state = cache.state.get(position)
            # what the step streams after this block: the next block's first matrix, or the output head
            if position + 1 < len(schedule):
                ctx.upcoming = self.blocks[schedule[position + 1].layer].mixer.first_weights()
            else:
                ctx.upcoming = kernels.next_weights(self.head) if ctx.n_wanted > 0 else None
            if block.fuses_next_norm:
                # the norm that reads this block's result, if its reader takes rows that lack their factor
                if position + 1 < len(schedule):
                    follower = self.blocks[schedule[position + 1].layer]
                    next_norm = follower.first_norm if follower.takes_scaled_pending else None
                else:
                    next_norm = self.final_norm if ctx.wants_every_row and ctx.n_wanted > 0 \
                        and self.final_norm is not None else None
                residual, pending = block.forward(residual, pending, ctx, view, state, next_norm=next_norm)
            else:
                residual, pending = block.forward(residual, pending, ctx, view, state)
        ctx.upcoming = None
        ctx.decode_plans = None
        if ctx.n_wanted == 0:
            return None
        if isinstance(pending, kernels.ScaledRows):
            return self._logits(pending)
        if not ctx.wants_every_row:
            residual = kernels.gather_rows(residual, ctx.wanted_rows)
            pending = kernels.gather_rows(pending, ctx.wanted_rows) if pending is not None else None
        if self.final_norm is None:
            return self._logits(residual if pending is None else kernels.add_rows(residual, pending))
        normed = self.final_norm.forward(residual) if pending is None else self.final_norm.add_forward(residual, pending)
        return self._logits(normed)

    def _logits(self, rows) -> torch.Tensor:
        """The output head, float32, with the architecture's factor and cap on the logits if it has them."""
        logits = kernels.linear(rows, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0 or self.spec.logit_softcap != 0.0:
            kernels.transform_logits(logits, self.spec.logit_scale, self.spec.logit_softcap)
        return logits
