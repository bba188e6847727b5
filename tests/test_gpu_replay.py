"""bin/trace_run driven as a user drives it: the same requests whole, with the last 32 tokens one
by one, and in batches of unequal lengths whose slots are used again, in both precisions."""

import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_model
from helpers import CONFIGS, assert_close, bf16_weights, prompts_for, write_model

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def replay(model, dtype, out, steps, max_tokens, graph):
    command = [str(ROOT / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
               "--max-tokens", str(max_tokens)]
    if graph != "default":
        command += ["--cuda-graph", graph]
    proc = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for record in steps:
        proc.stdin.write(json.dumps(record) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {record['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def read(out, step, vocab):
    return torch.from_numpy(np.fromfile(Path(out) / f"{step}.f32", dtype="<f4").reshape(-1, vocab))


@pytest.mark.parametrize("graph", ["default", "off"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_three_ways_of_cutting_the_same_requests(tmp_path, name, dtype, graph):
    """``graph`` default (on): single-token steps run on generation's fixed decode buffers through its CUDA
    graph and short prompt steps through the prompt graphs; off: every step launch by launch."""
    cfg = CONFIGS[name]
    weights = plain_model.random_weights(cfg, seed=91, matrix_std=0.06, norm_std=0.1)
    model = write_model(tmp_path / "model", cfg, weights)
    ref_w = weights if dtype == "float32" else bf16_weights(weights)
    requests = {f"r{i}": p for i, p in enumerate(prompts_for(cfg, [40, 33, 97, 64, 130, 35], seed=12))}
    want = {k: plain_model.forward(cfg, ref_w, p) for k, p in requests.items()}
    vocab = cfg["vocab_size"]

    # 1. each request alone and whole; every place wanted
    steps = [{"step": i, "entries": [{"id": k, "tokens": p, "want": list(range(len(p)))}], "end": [k]}
             for i, (k, p) in enumerate(requests.items())]
    replay(model, dtype, tmp_path / "whole", steps, 192, graph)
    for i, k in enumerate(requests):
        assert_close(read(tmp_path / "whole", i, vocab), want[k], dtype, f"whole {k}")

    # 2. all but the last 32 tokens whole, then one by one
    steps, expect, n = [], {}, 0
    for k, p in requests.items():
        head = len(p) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": p[:head], "want": [head - 1]}], "end": []})
        expect[n] = want[k][head - 1: head]
        n += 1
        for t in range(head, len(p)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [p[t]], "want": [0]}],
                          "end": [k] if t == len(p) - 1 else []})
            expect[n] = want[k][t: t + 1]
            n += 1
    replay(model, dtype, tmp_path / "tail", steps, 192, graph)
    for step, rows in expect.items():
        assert_close(read(tmp_path / "tail", step, vocab), rows, dtype, f"tail step {step}")

    # 3. batches of unequal lengths: prompts minus 5 tokens in one step, then one token each until the
    #    shorter ones are through; the next batch starts when the first has ended and takes its slots
    steps, expect, n = [], {}, 0
    names = list(requests)
    for batch in (names[:3], names[3:]):
        tails = {k: 3 + 2 * i for i, k in enumerate(batch)}
        steps.append({"step": n, "entries": [{"id": k, "tokens": requests[k][: -tails[k]],
                                              "want": [len(requests[k]) - tails[k] - 1]} for k in batch], "end": []})
        expect[n] = torch.stack([want[k][len(requests[k]) - tails[k] - 1] for k in batch])
        n += 1
        for t in range(max(tails.values())):
            live = [k for k in batch if t < tails[k]]
            steps.append({"step": n, "entries": [{"id": k, "tokens": [requests[k][len(requests[k]) - tails[k] + t]],
                                                  "want": [0] if t % 2 == 0 else []} for k in live],
                          "end": [k for k in live if t + 1 == tails[k]]})
            if t % 2 == 0:
                expect[n] = torch.stack([want[k][len(requests[k]) - tails[k] + t] for k in live])
            n += 1
    replay(model, dtype, tmp_path / "batches", steps, 64 + 64 + 128 + 64, graph)
    for step, rows in expect.items():
        assert_close(read(tmp_path / "batches", step, vocab), rows, dtype, f"batch step {step}")
    assert not (tmp_path / "batches" / "2.f32").exists()          # nothing wanted, nothing written
