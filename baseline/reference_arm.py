#!/usr/bin/env python3
"""Times the unmodified reference engine (M4cr0Chen/dryft-flash-infer, ``engine/engine.py``) on the
benchmark's decode step, in a process of its own.

    python baseline/reference_arm.py --model DIR --steps K --warmup W [--points] [--prefill] [--workloads]

``--model`` is a folder with ``config.json`` and ``model.safetensors`` in the checkpoint's tensor names (the
folder that ``python -m dryft_flash_infer_b200 random-model`` writes).  The reference is the copy of its
``engine/`` folder under ``baseline/_ref/engine``; it is imported the way its own harness imports it
(bench/harness.py:154-158: the folder on ``sys.path``, ``from engine import Engine``) and driven through its
public contract only: ``Engine(model_path)`` and ``generate(input_ids, max_new_tokens)``
(engine/engine.py:179-217, :1121-1157).  Nothing of this repository's package is imported here.

What is timed is what ``bench.py`` times for its own arm: batch 8, equal prompts, every sequence at the
benchmark context when the last timed step ends; a whole untimed ``generate`` of the same shape first (the
reference allocates, races its kernels and captures its graph at a shape's first call, engine/engine.py:360-490),
then W untimed decode steps inside the timed call, then K steps between two CUDA events on the stream the
reference replays its graph on (``value``), and the same steps by the wall clock with host lists in and
out (``e2e``).  The reference's stock settings decode with 8-bit weights wherever they win its warm-up
race (engine/engine.py:62); ``DRYFT_FP8=off`` in the environment gives its pure bfloat16 engine.

Prints one JSON object on the last line of standard output.
"""

from __future__ import annotations

import argparse
import io
import json
import os
import sys
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = ROOT / "baseline" / "_ref" / "engine"
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048


class _Tee(io.TextIOBase):
    """Passes the reference's stderr lines on and keeps those that say which path it took."""

    def __init__(self, under):
        self.under, self.kept = under, []

    def write(self, text):
        self.under.write(text)
        for line in text.splitlines():
            if line.startswith("engine:"):
                self.kept.append(line.strip())
        return len(text)

    def flush(self):
        self.under.flush()


def _prompts(batch: int, length: int, vocab: int, seed: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g).tolist()


def time_decode(engine, batch: int, context: int, steps: int, warmup: int, vocab: int):
    """(device ms per step, wall ms per step) of ``steps`` decode steps that end at ``context``."""
    import torch

    new = steps + warmup + 2
    length = context - new
    for _ in engine.generate(_prompts(batch, length, vocab, 1), new):       # the shape's first call: untimed
        pass
    torch.cuda.synchronize()
    stream = engine.generate(_prompts(batch, length, vocab, 2), new)
    for _ in range(1 + warmup):
        next(stream)
    # the stream runs one step ahead of its reader (engine/engine.py:1159-1185): warmup + 1 steps have been
    # launched by now, steps are left
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin = time.perf_counter()
    start.record()
    rows = sum(1 for _ in stream)
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - begin
    if rows != steps + 1:
        raise RuntimeError(f"the reference yielded {rows} rows where {steps + 1} were left")
    return start.elapsed_time(end) / steps, wall * 1e3 / steps


def time_prefill(engine, tokens: int, vocab: int):
    """Wall-clock milliseconds until the first token of one prompt of ``tokens`` tokens (upload included)."""
    import torch

    for _ in engine.generate(_prompts(1, tokens, vocab, 3), 2):
        pass
    times = []
    for seed in (4, 5, 6):
        prompt = _prompts(1, tokens, vocab, seed)
        torch.cuda.synchronize()
        begin = time.perf_counter()
        stream = engine.generate(prompt, 2)
        next(stream)
        torch.cuda.synchronize()
        times.append((time.perf_counter() - begin) * 1e3)
        for _ in stream:
            pass
    return sorted(times)[1]


#: the reference's own public workloads (bench/harness.py:26-30): name, batch, prompt tokens, output tokens
PUBLIC_WORKLOADS = (("public-0", 1, 512, 32), ("public-1", 4, 2048, 32), ("public-2", 16, 512, 128))


def time_workload(generate, batch: int, length: int, steps: int, vocab: int, samples: int = 5):
    """Generation as the reference's harness measures it (bench/harness.py:81-110): one untimed call, then
    ``samples`` calls by the wall clock; tokens/s = batch x output tokens / median seconds of a whole call
    (prefill included), TTFT the median time to the first row, TPOT the rest divided by the other rows."""
    import statistics

    import torch

    def once(seed):
        prompts = _prompts(batch, length, vocab, seed)
        torch.cuda.synchronize()
        begin = time.perf_counter()
        first, rows = None, 0
        for row in generate(prompts, steps):
            if first is None:
                first = time.perf_counter() - begin
            rows += 1
        torch.cuda.synchronize()
        total = time.perf_counter() - begin
        if rows != steps or len(row) != batch:
            raise RuntimeError(f"{rows} rows of {len(row)} tokens where {steps} of {batch} were asked for")
        return first, total

    once(100)
    records = [once(101 + i) for i in range(samples)]
    median = statistics.median(t for _, t in records)
    return {"tps": round(batch * steps / median, 1),
            "ttft_ms": round(statistics.median(f for f, _ in records) * 1e3, 2),
            "tpot_ms": round(statistics.median((t - f) / max(1, steps - 1) for f, t in records) * 1e3, 3)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", required=True)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--points", action="store_true", help="also batch 1 and 64, and the 512-token prompts")
    parser.add_argument("--prefill", action="store_true", help="also one prompt of 2,048 tokens")
    parser.add_argument("--workloads", action="store_true", help="also the reference's three public workloads")
    args = parser.parse_args()
    out: dict = {"impl": "reference", "settings": {k: v for k, v in os.environ.items() if k.startswith("DRYFT_")}}
    tee = _Tee(sys.stderr)
    sys.stderr = tee
    try:
        if not (REFERENCE / "engine.py").is_file():
            raise FileNotFoundError(f"no copy of the reference's engine folder at {REFERENCE}")
        sys.path.insert(0, str(REFERENCE))
        import torch
        from engine import Engine

        engine = Engine(args.model)
        out["fast_path_after_load"] = bool(engine._fast)
        vocab = json.loads((Path(args.model) / "config.json").read_text())["vocab_size"]
        ms, wall_ms = time_decode(engine, BATCH, CONTEXT, args.steps, args.warmup, vocab)
        out.update({"ms_per_step": round(ms, 4), "value": round(BATCH / ms * 1e3, 1),
                    "e2e_value": round(BATCH / wall_ms * 1e3, 1),
                    "decode_projections": {name: getattr(getattr(fn, "func", fn), "__name__", type(fn).__name__)
                                           for name, fn in (getattr(engine, "matmul", None) or {}).items()}})
        points = {}
        if args.points:
            quarter = max(8, args.steps // 4)
            for name, n, context, k in (("decode_b1", 1, CONTEXT, quarter), ("decode_b64", 64, CONTEXT, quarter),
                                        ("decode_b1_prompt512", 1, 512 + args.steps + args.warmup + 2, args.steps),
                                        ("decode_b8_prompt512", 8, 512 + args.steps + args.warmup + 2, args.steps),
                                        ("decode_b64_prompt512", 64, 512 + args.steps + args.warmup + 2, args.steps)):
                try:
                    point_ms, _ = time_decode(engine, n, context, k, args.warmup, vocab)
                    points[name] = round(n / point_ms * 1e3, 1)
                except Exception as exc:                      # one shape failing keeps the others
                    points[name] = f"failed: {type(exc).__name__}: {exc}"[:200]
        out["points"] = points
        if args.prefill:
            prefill_ms = time_prefill(engine, PREFILL_TOKENS, vocab)
            out["prefill"] = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                              "ms": round(prefill_ms, 3), "timed": "wall clock to the first token, upload included"}
        if args.workloads:
            out["workloads"] = {}
            for name, batch, length, steps in PUBLIC_WORKLOADS:
                try:
                    out["workloads"][name] = time_workload(engine.generate, batch, length, steps, vocab)
                except Exception as exc:
                    out["workloads"][name] = f"failed: {type(exc).__name__}: {exc}"[:200]
        out["fast_path"] = bool(engine._fast)
        torch.cuda.synchronize()
    except Exception as exc:
        traceback.print_exc()
        out["unavailable"] = f"{type(exc).__name__}: {exc}"[:400]
    finally:
        sys.stderr = tee.under
    out["engine_lines"] = tee.kept[-12:]
    out["fell_back_to_native"] = any("native" in line for line in tee.kept)
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
