"""The plain implementation against the reference's own CPU output (tests/golden)."""

from pathlib import Path

import numpy as np
import torch

import plain_model

GOLDEN = Path(__file__).resolve().parent / "golden"


def _load(name, cfg):
    data = np.load(GOLDEN / f"{name}.npz")
    weights = plain_model.random_weights(cfg, int(data["seed"]))
    checksum = float(sum(t.double().abs().sum() for t in weights.values()))
    assert abs(checksum - float(data["weight_checksum"])) < 1e-6 * checksum, "seeded weights changed"
    return data, weights


def test_tied_logits_match_reference_cpu_code():
    cfg = plain_model.TINY_A
    data, weights = _load("tiny_a_reference", cfg)
    head = weights["model.embed_tokens.weight"]
    for row, ids in enumerate(data["ids"]):
        want = torch.from_numpy(data["final_hidden"][row]) @ head.T
        got = plain_model.forward(cfg, weights, ids.tolist())
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), float((got - want).abs().max())


def test_untied_logits_match_reference_cpu_code():
    cfg = plain_model.TINY_B
    data, weights = _load("tiny_b_reference", cfg)
    head = weights["lm_head.weight"]
    for row, ids in enumerate(data["ids"]):
        want = torch.from_numpy(data["final_hidden"][row]) @ head.T
        got = plain_model.forward(cfg, weights, ids.tolist())
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), float((got - want).abs().max())


def test_greedy_tokens_match_reference_cached_decode():
    cfg = plain_model.TINY_A
    data, weights = _load("tiny_a_reference", cfg)
    greedy = data["greedy"]  # [steps, batch]
    for row, ids in enumerate(data["ids"]):
        got = plain_model.greedy_continue(cfg, weights, ids.tolist(), greedy.shape[0])
        assert got == greedy[:, row].tolist()


def test_parts_alone():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    y = plain_model.rms_norm(x, w, 1e-5)
    assert torch.allclose((y / w).pow(2).mean(-1), torch.ones(5), atol=1e-3)
    # a rotation keeps lengths, and position 0 is the identity
    v = torch.randn(4, 3, 8)
    ang = plain_model.rope_angles(torch.arange(4), 8, 100.0)
    r = plain_model.apply_rope(v, ang)
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1), atol=1e-5)
    assert torch.allclose(r[0], v[0])
    # a window of 1 attends to the token itself only
    q, k, val = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain_model.causal_attention(q, k, val, window=1)
    assert torch.allclose(out, val.repeat_interleave(2, dim=1), atol=1e-6)
    # the first token of causal attention sees itself only
    out = plain_model.causal_attention(q, k, val)
    assert torch.allclose(out[0], val[0].repeat_interleave(2, dim=0), atol=1e-6)


def test_sampling_formula():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    p = plain_model.temperature_probabilities(logits, 0.5)
    assert abs(float(p.sum()) - 1) < 1e-12
    assert plain_model.sample_from_uniform(p, 0.0) == 0
    assert plain_model.sample_from_uniform(p, 0.999999) == 3        # p[3] = 0.0021: the last 0.2 % of the line
    cdf = torch.cumsum(p, 0)
    assert plain_model.sample_from_uniform(p, float(cdf[1]) - 1e-9) == 1
    assert plain_model.sample_from_uniform(p, float(cdf[1]) + 1e-9) == 2
