"""Grouped-query attention over the paged cache: the mixer of the Qwen3 decoder."""

from __future__ import annotations

from ..ops import kernels
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part
from .spec import PartSpec


class Attention(Mixer):
    """``o_proj(attend(rope(q_norm(q)), rope(k_norm(k)), v))`` with no biases.

    q, k and v come from one fused matrix ``[n_q*D + 2*n_kv*D, hidden]`` (q rows, then k,
    then v: engine/engine.py:163-168).  Each head of q and k is RMS-normalised with a
    weight shared by all heads, then rotated (engine/kernels/reference.py:31-46); v gets
    neither.  Keys and values are written into the cache at each token's position and
    the queries attend causally over their sequence's cache, query head ``h`` reading
    key/value head ``h // (n_q / n_kv)``, scores scaled by ``scale`` (default
    ``head_dim ** -0.5``, engine/kernels/attention.py:210).  ``window`` > 0 limits each
    query to the latest ``window`` keys.  ``qk_norm`` and ``position`` may be absent.

    What the mixer asks of its position part: float32 tables ``cos`` and ``sin`` of shape
    ``[positions, r / 2]`` with ``r <= head_dim`` even, made by ``prepare``; element ``i < r / 2`` of a
    head is rotated with element ``i + r / 2`` by the angle whose cosine and sine stand at ``[position,
    i]``, and elements from ``r`` on are left as they are.
    """

    kind = "attention"
    accepts_scaled_rows = True
    fuses_add_norm = True

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, qk_norm: bool = True,
                 qk_norm_eps: float = 1e-6, position: PartSpec | None = None, window: int = 0,
                 scale: float | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"attention takes head sizes in steps of 16 up to 256, got {head_dim}")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.qk_norm, self.qk_norm_eps, self.window = qk_norm, float(qk_norm_eps), int(window)
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.position = build_part("position", position, hidden_size) if position is not None else None
        self.qkv = self.o = self.q_norm = self.k_norm = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def tensors(self):
        q_rows, kv_rows = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = {
            "q_proj": TensorDecl((q_rows, self.hidden_size), "qkv", 0),
            "k_proj": TensorDecl((kv_rows, self.hidden_size), "qkv", q_rows),
            "v_proj": TensorDecl((kv_rows, self.hidden_size), "qkv", q_rows + kv_rows),
            "o_proj": TensorDecl((self.hidden_size, q_rows), "o"),
        }
        if self.qk_norm:
            out["q_norm"] = TensorDecl((self.head_dim,), "q_norm", init="norm", precision="float32")
            out["k_norm"] = TensorDecl((self.head_dim,), "k_norm", init="norm", precision="float32")
        return out

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def prepare(self, max_positions: int, device) -> None:
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def first_weights(self):
        return kernels.next_weights(self.qkv)

    def forward(self, x, ctx, cache, state, add_norm=None):
        qkv = kernels.linear(x, self.qkv)
        cos = self.position.cos if self.position is not None else None
        sin = self.position.sin if self.position is not None else None
        if kernels.decode_prepares_tokens(qkv, ctx, self.n_heads, self.n_kv_heads, self.head_dim, cos):
            # decoding: the attention kernel normalises, rotates and stores the new token itself
            prep = kernels.TokenPrep(qkv, self.q_norm, self.k_norm, self.qk_norm_eps, cos, sin)
            attended = kernels.attention_decode(None, cache, ctx, self.n_heads, self.n_kv_heads, self.head_dim,
                                                self.scale, self.window, prep=prep)
            return kernels.linear(attended, self.o, add_norm=add_norm, then=getattr(ctx, "upcoming", None))
        q = kernels.qk_norm_rope_write(qkv, self.n_heads, self.n_kv_heads, self.head_dim, self.q_norm, self.k_norm,
                                       self.qk_norm_eps, cos, sin, ctx.row_pos, ctx.row_seq, cache)
        attended = kernels.attention(q, cache, ctx, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                     self.window)
        return kernels.linear(attended, self.o, add_norm=add_norm, then=getattr(ctx, "upcoming", None))


register_part("mixer", Attention.kind, Attention)
