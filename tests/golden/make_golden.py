"""Makes ``tests/golden/*.npz``: logits of the reference's own CPU code on tiny random models.

Run once, with the reference project's ``engine/`` folder given on the command line:

    python tests/golden/make_golden.py /path/to/reference/engine

The reference's ``Engine`` is built without its loader (``Engine.__new__``) around a
namespace tree that holds our seeded random weights, with Triton made unimportable so
that its kernel package takes the plain-torch branch (engine/kernels/__init__.py:11-37).
Its ``_blocks`` then runs in float32 on the CPU once the two bfloat16-typed pieces of
state (RoPE tables, cache) are replaced by float32 ones.  No model code of any
installed package is involved.

Limits of the anchor: the reference wants equal prompt lengths and tied embeddings
(engine/engine.py:233-234, :1133).  For the untied configuration the final normed
hidden state is stored and the test applies the separate head by formula.  Sampling
with a temperature has no counterpart in the reference and rests on formulas alone.
"""

from __future__ import annotations

import sys
from pathlib import Path
from types import SimpleNamespace as NS

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_model  # noqa: E402


def reference_engine(engine_dir: str, cfg: dict, weights: dict):
    sys.modules["triton"] = None
    if engine_dir not in sys.path:
        sys.path.insert(0, engine_dir)
    import engine as E

    def lin(name):
        return NS(weight=weights[name])

    layers = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layers.append(NS(
            self_attn=NS(q_proj=lin(p + "self_attn.q_proj.weight"), k_proj=lin(p + "self_attn.k_proj.weight"),
                         v_proj=lin(p + "self_attn.v_proj.weight"), o_proj=lin(p + "self_attn.o_proj.weight"),
                         q_norm=lin(p + "self_attn.q_norm.weight"), k_norm=lin(p + "self_attn.k_norm.weight")),
            input_layernorm=lin(p + "input_layernorm.weight"),
            post_attention_layernorm=lin(p + "post_attention_layernorm.weight"),
            mlp=NS(gate_proj=lin(p + "mlp.gate_proj.weight"), up_proj=lin(p + "mlp.up_proj.weight"),
                   down_proj=lin(p + "mlp.down_proj.weight"))))
    fake = NS(
        config=NS(hidden_size=cfg["hidden_size"], num_attention_heads=cfg["num_attention_heads"],
                  num_key_value_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                  num_hidden_layers=cfg["num_hidden_layers"], rms_norm_eps=cfg["rms_norm_eps"],
                  rope_theta=cfg["rope_theta"], tie_word_embeddings=True),
        model=NS(embed_tokens=lin("model.embed_tokens.weight"), norm=lin("model.norm.weight"), layers=layers))
    eng = E.Engine.__new__(E.Engine)
    eng.cuda, eng.device, eng._native, eng._fast = False, "cpu", None, True
    eng._adopt(fake)
    return E, eng


def to_float32_state(E, eng, batch, seq_len, steps):
    capture = E.Engine._capture
    E.Engine._capture = lambda self: None
    eng._ensure(batch, seq_len, steps)
    E.Engine._capture = capture
    half = eng.head_dim // 2
    inv = 1.0 / (eng.rope_theta ** (torch.arange(0, half).float() / half))
    emb = torch.cat([torch.arange(eng.capacity).float()[:, None] * inv[None, :]] * 2, -1)
    eng.cos, eng.sin = emb.cos().contiguous(), emb.sin().contiguous()
    eng.k_cache = torch.zeros_like(eng.k_cache, dtype=torch.float32)
    eng.v_cache = torch.zeros_like(eng.k_cache)


def make(engine_dir: str, name: str, cfg: dict, seed: int, batch: int, seq_len: int, steps: int):
    import torch.nn.functional as F

    weights = plain_model.random_weights(cfg, seed)
    E, eng = reference_engine(engine_dir, plain_model.normalise_config(cfg), weights)
    to_float32_state(E, eng, batch, seq_len, steps)
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, cfg["vocab_size"], (batch, seq_len), generator=g)
    with torch.no_grad():
        x = F.embedding(ids, eng.embed).view(batch * seq_len, cfg["hidden_size"])
        normed = eng._blocks(x, eng.arange[:seq_len], seq_len, batch, 0, eng._attend_prefill)
        tokens = []
        if cfg["tie_word_embeddings"]:
            eng._prefill(ids)
            tokens.append(eng.emitted.tolist())
            for _ in range(steps - 1):
                eng._decode_step()
                tokens.append(eng.emitted.tolist())
    checksum = float(sum(t.double().abs().sum() for t in weights.values()))
    np.savez_compressed(
        HERE / f"{name}.npz",
        ids=ids.numpy(), final_hidden=normed.view(batch, seq_len, -1).numpy(),
        greedy=np.array(tokens, dtype=np.int64), seed=np.int64(seed), weight_checksum=np.float64(checksum))
    print(name, "final_hidden", tuple(normed.shape), "greedy", tokens)


if __name__ == "__main__":
    engine_dir = sys.argv[1]
    make(engine_dir, "tiny_a_reference", plain_model.TINY_A, seed=11, batch=3, seq_len=9, steps=8)
    make(engine_dir, "tiny_b_reference", plain_model.TINY_B, seed=23, batch=2, seq_len=11, steps=4)
