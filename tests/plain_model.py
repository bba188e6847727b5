"""A plain, slow implementation of the Qwen3 dense decoder for the tests.

Whole sequences only, no cache, float32 (or float64) on the CPU, one function
for each part.  It shares no code with the package: every function below is
written from the formulas of the reference engine, whose file and line it
cites (paths are relative to the reference project).  Where the reference
rounds to bfloat16 between operations, this implementation keeps full
precision: it is the exact arithmetic that both of the engine's precisions
are compared with.

``tests/golden/`` holds logits that the reference's own CPU code produced for a
tiny random model; ``tests/test_plain_model.py`` checks this file against them.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- parts


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """``x = E[ids]`` (engine/engine.py:1019, :1037)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last axis
    (engine/kernels/reference.py:13-16; the bfloat16 rounding there is left out)."""
    scale = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * scale * weight


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """Rotation angles ``[len(positions), head_dim]``, float32 as the reference builds them:
    ``inv_freq_i = 1 / theta^(i / half)``, ``angle = cat(p * inv_freq, p * inv_freq)``
    (engine/engine.py:350-356)."""
    half = head_dim // 2
    steps = torch.arange(0, half, dtype=torch.int64).float()
    inv_freq = 1.0 / (theta ** (steps / half))
    p = positions.to(torch.int64).float()
    return torch.cat([p[:, None] * inv_freq[None, :]] * 2, dim=-1)


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of ``x [tokens, heads, head_dim]``:
    ``x * cos + cat(-x[half:], x[:half]) * sin`` (engine/kernels/reference.py:31-46)."""
    half = x.shape[-1] // 2
    cos = angles.cos().to(x.dtype)[:, None, :]
    sin = angles.sin().to(x.dtype)[:, None, :]
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rotated * sin


def head_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMSNorm of ``x [tokens, heads, head_dim]`` with one weight vector
    for all heads (engine/kernels/reference.py:36-38)."""
    return rms_norm(x, weight, eps)


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float | None = None,
    window: int = 0,
) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.

    ``q [T, Nq, D]``, ``k, v [T, Nkv, D]``; query head ``h`` reads key/value head
    ``h // (Nq // Nkv)``; scores ``q.k / sqrt(D)``, mask ``j <= i``, float32 softmax
    (engine/engine.py:964-982; the grouping and the scale are spelled out in
    engine/kernels/attention.py:40-137 and :210).  ``window`` > 0 also hides keys
    with ``j <= i - window``; the reference has no window and the Qwen3 tests
    leave it at 0.
    """
    tokens, n_q, dim = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    if scale is None:
        scale = dim ** -0.5
    out = torch.empty_like(q)
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    hidden = j > i
    if window > 0:
        hidden = hidden | (j <= i - window)
    for head in range(n_q):
        scores = (q[:, head, :] @ k[:, head // group, :].T) * scale
        scores = scores.masked_fill(hidden, -math.inf)
        probs = torch.softmax(scores, dim=-1)
        out[:, head, :] = probs @ v[:, head // group, :]
    return out


def attention_block(x, w, prefix, cfg, positions, window: int = 0):
    """q/k/v projections without bias, per-head q_norm/k_norm, RoPE on q and k,
    attention, output projection (engine/engine.py:163-171, :933-949)."""
    n_q, n_kv, dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    tokens = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(tokens, n_q, dim)
    k = (x @ w[prefix + "k_proj.weight"].T).view(tokens, n_kv, dim)
    v = (x @ w[prefix + "v_proj.weight"].T).view(tokens, n_kv, dim)
    q = head_norm(q, w[prefix + "q_norm.weight"], eps)
    k = head_norm(k, w[prefix + "k_norm.weight"], eps)
    angles = rope_angles(positions, dim, cfg["rope_theta"])
    q = apply_rope(q, angles)
    k = apply_rope(k, angles)
    att = causal_attention(q, k, v, window=window).reshape(tokens, n_q * dim)
    return att @ w[prefix + "o_proj.weight"].T


def swiglu_mlp(x, w, prefix):
    """``down(silu(gate(x)) * up(x))`` with ``silu(g) = g / (1 + exp(-g))``
    (engine/engine.py:173-176, :950-961; engine/kernels/reference.py:74-79)."""
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    inner = gate / (1.0 + torch.exp(-gate)) * up
    return inner @ w[prefix + "down_proj.weight"].T


def decoder_layer(x, w, index, cfg, positions, window: int = 0):
    """Pre-norm block: ``x += attn(norm(x))``, ``x += mlp(norm(x))``
    (the residual chain of engine/engine.py:918-961 written without fusion)."""
    p = f"model.layers.{index}."
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(
        rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, positions, window
    )
    x = x + swiglu_mlp(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return x


# --------------------------------------------------------------------------- model


def normalise_config(cfg: dict) -> dict:
    """The numbers the formulas need, with the reference's defaults
    (engine/engine.py:223-234: head_dim defaults to hidden // heads)."""
    out = dict(cfg)
    out.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    out.setdefault("rms_norm_eps", 1e-6)
    out.setdefault("tie_word_embeddings", False)
    return out


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, windows=None, places=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` at every position of one sequence (or ``[len(places), vocab]`` at the
    positions ``places``: the head is a large product when the vocabulary is).

    embed -> layers -> final norm -> head, the head being the embedding table when
    ``tie_word_embeddings`` (engine/engine.py:236-239, :1019-1025).  ``windows``
    optionally gives a window per layer (0 = all keys).
    """
    cfg = normalise_config(cfg)
    w = {name: t.to(dtype) for name, t in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.int64)
    positions = torch.arange(ids.numel())
    x = embedding(w["model.embed_tokens.weight"], ids)
    for index in range(cfg["num_hidden_layers"]):
        window = windows[index] if windows else 0
        x = decoder_layer(x, w, index, cfg, positions, window)
    if places is not None:
        x = x[torch.as_tensor(list(places), dtype=torch.int64)]
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def greedy_continue(cfg: dict, weights: dict, prompt, steps: int, dtype=torch.float32):
    """Greedy continuation by running the whole sequence again for every token;
    argmax takes the lowest index on ties (engine/engine.py:1026, :1046)."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(cfg, weights, seq, dtype)[-1]
        token = int(torch.argmax(logits))
        out.append(token)
        seq.append(token)
    return out


# --------------------------------------------------------------------------- sampling


def temperature_probabilities(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``softmax(logits / temperature)`` in float64.  The reference only takes the
    argmax (engine/engine.py:1026); temperature sampling rests on this formula alone."""
    return torch.softmax(logits.double() / temperature, dim=-1)


def sample_from_uniform(probs: torch.Tensor, u: float) -> int:
    """Inverse CDF: the first index whose cumulative probability exceeds ``u``."""
    cdf = torch.cumsum(probs.double(), dim=-1)
    index = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64), right=True))
    return min(index, probs.numel() - 1)


# --------------------------------------------------------------------------- random models


def random_weights(cfg: dict, seed: int, matrix_std: float = 0.02, norm_std: float = 0.01) -> dict:
    """A float32 state dict with the tensor names of the architecture: matrices
    N(0, matrix_std), norm weights 1 + N(0, norm_std)."""
    cfg = normalise_config(cfg)
    g = torch.Generator().manual_seed(seed)
    hidden, inter, vocab = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    n_q, n_kv, dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(rows, cols):
        return torch.randn(rows, cols, generator=g) * matrix_std

    def vec(n):
        return 1.0 + norm_std * torch.randn(n, generator=g)

    w = {"model.embed_tokens.weight": mat(vocab, hidden), "model.norm.weight": vec(hidden)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = vec(hidden)
        w[p + "post_attention_layernorm.weight"] = vec(hidden)
        w[p + "self_attn.q_proj.weight"] = mat(n_q * dim, hidden)
        w[p + "self_attn.k_proj.weight"] = mat(n_kv * dim, hidden)
        w[p + "self_attn.v_proj.weight"] = mat(n_kv * dim, hidden)
        w[p + "self_attn.o_proj.weight"] = mat(hidden, n_q * dim)
        w[p + "self_attn.q_norm.weight"] = vec(dim)
        w[p + "self_attn.k_norm.weight"] = vec(dim)
        w[p + "mlp.gate_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.up_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.down_proj.weight"] = mat(hidden, inter)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(vocab, hidden)
    return w


TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "hidden_act": "silu",
    "max_position_embeddings": 4096, "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 320, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
    "max_position_embeddings": 4096, "torch_dtype": "float32",
}
