#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-4B sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 with every
sequence at the benchmark context length (the last timed step ends there), timed on the
device over K decode steps (default 256, the benchmark configuration's generated tokens) after W
warm-up steps (each step launched before the tokens of the step before it are read, as generation does).  ``e2e`` is the same through
``Engine.generate`` with host token lists in and out.  ``prefill`` is one prompt of 2,048
tokens; ``points`` are decode at batch 1 and 64 at that context, and at batch 1, 8 and 64 right after
prompts of 512 tokens; ``roofline`` compares the bytes a decode
step has to read (every weight once, the live requests' cache) with the HBM peak.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the sizes of Qwen3-4B (36 layers, hidden 2560, 32/8 heads of 128, intermediate 9728, vocabulary 151936)
QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# the sizes of Qwen3-8B and Qwen3-14B, for the end-to-end generation runs of --shape
QWEN3_8B = dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, rope_theta=1000000.0, tie_word_embeddings=False)
QWEN3_14B = dict(QWEN3_4B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408,
                 rope_theta=1000000.0, tie_word_embeddings=False)
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
PROMPT_OF_POINTS = 512      # the prompts of the benchmark configuration's decode runs
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz, top, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7 or not parts[0].isdigit():
                continue
            mhz.append(int(parts[0]))
            top = max(top, int(parts[1]))
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": top or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_numbers(cfg: dict, layers: int) -> dict:
    h, inter, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nq, nkv, vocab = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    per_layer = (nq + 2 * nkv) * d * h + h * nq * d + 3 * inter * h
    return {"layer_params": per_layer, "weight_bytes": 2 * (layers * per_layer + vocab * h),
            "kv_bytes_per_token": 2 * 2 * nkv * d * layers, "head_params": vocab * h}


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    nums = model_numbers(cfg, layers)
    linear = 2.0 * tokens * layers * nums["layer_params"]
    attention = layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * tokens / 2
    return linear + attention + 2.0 * nums["head_params"]


def fill_context(engine, n_seqs: int, length: int):
    """Opens ``n_seqs`` slots holding ``length`` tokens each of synthetic keys and values."""
    slots = []
    for _ in range(n_seqs):
        slot = engine.open_slot()
        engine.cache.book.reserve(slot, length)
        engine.cache.book.advance(slot, length)
        slots.append(slot)
    return slots


def time_decode(engine, n_seqs: int, context: int, steps: int, warmup: int, sampler=None):
    import torch
    from dryft_flash_infer_b200.ops import kernels
    from dryft_flash_infer_b200.sampling import SamplingParams

    params = SamplingParams()
    slots = fill_context(engine, n_seqs, context - steps - warmup - 1)
    tokens = [(17 * i + 3) % engine.config.vocab_size for i in range(n_seqs)]
    # as in generation, a step is launched before the tokens of the step before it are read: it is fed on
    # the device, and the host's turn-around hides behind the running step
    ids = list(range(n_seqs))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = kernels.LAUNCHES
    handle = None
    for i in range(warmup + steps):
        if i == warmup:
            launches_before = kernels.LAUNCHES
            start.record()
        launched = engine.decode_launch(slots, tokens if i == 0 else None, ids, 1 + i, params)
        if handle is not None:
            handle.result()
        handle = launched
    end.record()
    handle.result()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    batch = next(iter(b for b in engine.decoder.batches.values() if b.n >= n_seqs))
    per_step = batch.launches_per_step if batch.graph else (kernels.LAUNCHES - launches_before) // max(1, steps)
    for slot in slots:
        engine.close_slot(slot)
    return ms, per_step


#: the reference's public workloads (bench/harness.py:26-30): name, batch, prompt tokens, output tokens
PUBLIC_WORKLOADS = (("public-0", 1, 512, 32), ("public-1", 4, 2048, 32), ("public-2", 16, 512, 128))


def time_workload(engine, batch: int, length: int, steps: int, vocab: int, g, samples: int = 5) -> dict:
    """A whole ``Engine.generate`` call as the reference's harness times it (bench/harness.py:81-110): one untimed
    call, then ``samples`` by the wall clock with host token lists in and out; tokens/s = batch x output tokens /
    median seconds (prefill included), TTFT = median time to the first row, TPOT = the rest per further row."""
    import torch

    def once():
        prompts = [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(batch)]
        torch.cuda.synchronize()
        begin = time.perf_counter()
        first, rows = None, 0
        for _ in engine.generate(prompts, steps):
            if first is None:
                first = time.perf_counter() - begin
            rows += 1
        torch.cuda.synchronize()
        assert rows == steps
        return first, time.perf_counter() - begin

    once()
    records = [once() for _ in range(samples)]
    median = statistics.median(t for _, t in records)
    return {"tps": round(batch * steps / median, 1),
            "ttft_ms": round(statistics.median(f for f, _ in records) * 1e3, 2),
            "tpot_ms": round(statistics.median((t - f) / max(1, steps - 1) for f, t in records) * 1e3, 3)}


def long_engine(engine, context: int):
    """``engine`` with its cache made anew for one sequence of ``context`` tokens (the weights stay)."""
    engine._make_cache(context, 1, context)
    for group in engine.cache.groups:
        group.k.normal_(0.0, 1.0)
        group.v.normal_(0.0, 1.0)
    return engine


def generation_run(shape: str) -> int:
    """Generation through ``Engine.generate`` at the 8B shape (16 unequal prompts of 128..2,048 tokens, 256
    greedy steps) or the 14B shape (32 prompts of 1,024 tokens, 128 steps): tokens per second, prefill included."""
    import torch
    from dryft_flash_infer_b200 import Engine

    cfg, batch, new = (QWEN3_8B, 16, 256) if shape == "8b" else (QWEN3_14B, 32, 128)
    g = torch.Generator().manual_seed(1)
    if shape == "8b":
        lengths = torch.randint(128, 2049, (batch,), generator=g).tolist()
    else:
        lengths = [1024] * batch
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    engine = Engine(config=cfg, random_weights=True, seed=0, dtype="bfloat16")
    list(engine.generate([p[:64] for p in prompts[:batch]], 4))            # warm-up: compiles nothing new, builds graphs
    results = []
    for _ in range(2):
        torch.cuda.synchronize()
        begin = time.perf_counter()
        stream = engine.generate(prompts, new)
        next(stream)
        torch.cuda.synchronize()
        first = time.perf_counter()
        produced = 1 + sum(1 for _ in stream)
        torch.cuda.synchronize()
        end = time.perf_counter()
        results.append((end - begin, first - begin, produced))
    total, ttft, produced = min(results)
    nums = model_numbers(cfg, cfg["num_hidden_layers"])
    peak = peaks()
    tpot = (total - ttft) / max(1, produced - 1)
    # a decode step reads every weight once and the cache of the live sequences (on average half the new tokens in)
    step_bytes = nums["weight_bytes"] + (sum(lengths) + batch * produced / 2) * nums["kv_bytes_per_token"]
    achieved = step_bytes / tpot / 1e9
    flops = sum(prefill_flops(cfg, cfg["num_hidden_layers"], n) for n in lengths)      # each prompt: its products, its own causal attention, one head row
    print(json.dumps({
        "metric": f"generation tokens/s, prefill included (Qwen3-{shape.upper()} sizes, bf16, random weights)",
        "value": round(batch * produced / total, 1), "unit": "tokens/s", "n_gpus": 1, "impl": "ours",
        "ttft_ms": round(ttft * 1e3, 2), "tpot_ms": round((total - ttft) / max(1, produced - 1) * 1e3, 3),
        "prefill_tokens_per_s": round(sum(lengths) / ttft, 1),
        "prefill": {"value": round(sum(lengths) / ttft, 1), "tokens": sum(lengths), "ms": round(ttft * 1e3, 2),
                    "frac": round(flops / ttft / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"],
                     "bytes_per_step_gb": round(step_bytes / 1e9, 2)},
        "config": {"model": f"Qwen3-{shape.upper()} sizes", "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "prompt_tokens": sum(lengths), "new_tokens": produced, "weight_gb": round(nums["weight_bytes"] / 1e9, 2)},
        "data": "synthetic: random weights, random token ids"}))
    return 0


def headline_config(layers: int) -> dict:
    cfg = QWEN3_4B
    return {"model": "Qwen3-4B sizes", "layers": layers, "layers_of_config": cfg["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": BATCH, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "parallelism": "none",
            "cuda_graph": True, "l2": "weights read per step (8 GB) exceed L2 (126 MB)"}


def reference_run(steps: int, warmup: int, quick: bool) -> int:
    """The reference arm: the unmodified reference engine (its ``engine/`` folder copied to
    ``baseline/_ref/engine``) on the headline's decode step, through ``Engine(model_path).generate``.

    This process only writes the model folder (Qwen3-4B sizes, random weights, this package's writer) and
    starts ``baseline/reference_arm.py`` twice, in processes of their own because the reference reads its
    settings from the environment at import: once with its stock settings (8-bit decode weights where
    they win its warm-up race) and once with ``DRYFT_FP8=off`` (its pure bfloat16 engine)."""
    import os
    import tempfile

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    arm = ROOT / "baseline" / "reference_arm.py"
    if not (ROOT / "baseline" / "_ref" / "engine" / "engine.py").is_file():
        return unavailable("no copy of the reference under baseline/_ref/engine (copy its engine/ folder there; "
                           "pip cannot install it: it has neither setup.py nor pyproject.toml)")
    try:
        import torch
        from dryft_flash_infer_b200.config import config_from_dict
        from dryft_flash_infer_b200.weights import write_random_model

        if not torch.cuda.is_available():
            return unavailable("no CUDA device is visible")
        with tempfile.TemporaryDirectory(prefix="dfi_reference_model_") as folder:
            print("reference arm: writing a Qwen3-4B-sized random model folder", file=sys.stderr, flush=True)
            write_random_model(config_from_dict(QWEN3_4B), 0, folder, torch.bfloat16, device="cuda:0")
            torch.cuda.empty_cache()
            results = {}
            with ClockSampler() as clocks:
                for name, env, extra in (("stock", {}, [] if quick else ["--points", "--prefill", "--workloads"]),
                                         ("bf16", {"DRYFT_FP8": "off"}, [] if quick else ["--workloads"])):
                    environment = {k: v for k, v in os.environ.items() if not k.startswith("DRYFT_")}
                    environment.update(env)
                    print(f"reference arm: running the reference with {env or 'its stock settings'}", file=sys.stderr,
                          flush=True)
                    done = subprocess.run([sys.executable, str(arm), "--model", folder, "--steps", str(steps),
                                           "--warmup", str(warmup), *extra], env=environment, stdout=subprocess.PIPE,
                                          text=True, timeout=1500)
                    lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
                    if done.returncode != 0 or not lines:
                        results[name] = {"unavailable": f"the reference's process ended with code {done.returncode} "
                                                        f"and no result line"}
                    else:
                        results[name] = json.loads(lines[-1])
    except Exception as exc:                                   # noqa: BLE001 - the arm reports, it does not raise
        return unavailable(f"{type(exc).__name__}: {exc}"[:400])
    stock, bf16 = results["stock"], results["bf16"]
    if "unavailable" in stock:
        return unavailable(f"the reference raised on this image: {stock['unavailable']}; "
                           f"its last lines: {' | '.join(stock.get('engine_lines', []))}"[:600])
    path = "the reference's own engine" if stock.get("fast_path") and not stock.get("fell_back_to_native") \
        else "NOT the reference's engine: it fell back to its native Transformers loop"
    line = {
        "metric": "decode tokens/s at batch 8 (Qwen3-4B sizes, bf16, random weights)",
        "value": stock["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": stock["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids", "impl": "reference",
        "path": path, "weights_of_decode_products": stock.get("decode_projections"),
        "config": headline_config(QWEN3_4B["num_hidden_layers"]),
        "e2e": {"value": stock["e2e_value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": BATCH * 8},
        "bf16_weights": ({"value": bf16["value"], "ms_per_step": bf16["ms_per_step"], "e2e_value": bf16["e2e_value"],
                          "fast_path": bf16.get("fast_path"), "settings": bf16.get("settings"),
                          "workloads": bf16.get("workloads")}
                         if "unavailable" not in bf16 else {"unavailable": bf16["unavailable"]}),
        "points": stock.get("points", {}), "prefill": stock.get("prefill"), "workloads": stock.get("workloads"),
        "engine_lines": stock.get("engine_lines", [])[-6:], "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256,
                        help="timed decode steps (default: the 256 generated tokens of the benchmark configuration)")
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=QWEN3_4B["num_hidden_layers"],
                        help="fewer layers than the configuration has (both numbers are reported)")
    parser.add_argument("--quick", action="store_true", help="skip the batch 1/64 points and the end-to-end run")
    parser.add_argument("--profile", choices=["decode", "prefill", "timeline"],
                        help="run only a few plain (graph-less) decode steps or one prefill, for a profiler; prints no JSON")
    parser.add_argument("--batch", type=int, default=BATCH, help="batch of the --profile decode steps")
    parser.add_argument("--context", type=int, default=CONTEXT, help="context length of the --profile decode steps")
    parser.add_argument("--shape", choices=["4b", "8b", "14b"], default="4b",
                        help="8b / 14b: the end-to-end generation runs of the larger shapes instead of the headline run")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run it with --gpus 1")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.impl == "reference":
        return reference_run(steps, warmup, args.quick)
    if args.shape != "4b":
        return generation_run(args.shape)

    import torch
    from dryft_flash_infer_b200 import Engine, StepEntry

    cfg = dict(QWEN3_4B, num_hidden_layers=args.layers)
    nums = model_numbers(cfg, args.layers)
    peak = peaks()
    max_seqs = 64
    engine = Engine(config=cfg, random_weights=True, seed=0, dtype="bfloat16", max_tokens=max_seqs * CONTEXT,
                    max_seqs=max_seqs, max_context=CONTEXT)
    for group in engine.cache.groups:            # synthetic cache content, the same for every run
        group.k.normal_(0.0, 1.0)
        group.v.normal_(0.0, 1.0)
    g = torch.Generator().manual_seed(0)
    if args.profile == "decode":
        engine.decoder.use_graph = False
        ms, launches = time_decode(engine, args.batch, args.context, steps, warmup)
        print(f"profile run: {steps} plain decode steps at batch {args.batch} and context {args.context}, {ms:.3f} ms and "
              f"{launches} launches per step")
        return 0
    if args.profile == "timeline":
        # kernel records of one graph replay: when each kernel of a layer ends after the one before it
        from torch.profiler import ProfilerActivity, profile
        from dryft_flash_infer_b200.sampling import SamplingParams

        slots = fill_context(engine, args.batch, args.context - 64)
        tokens = [3] * args.batch
        for i in range(5):
            tokens = engine.decode(slots, tokens, list(range(args.batch)), 1 + i, SamplingParams())
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(3):
                tokens = engine.decode(slots, tokens, list(range(args.batch)), 10 + i, SamplingParams())
            torch.cuda.synchronize()
        events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                        key=lambda e: e.time_range.end)
        marks = [i for i, e in enumerate(events) if "argmax" in e.name]
        step = events[marks[0] + 1: marks[1] + 1]
        kernels_only = [e for e in step if "Memcpy" not in e.name]
        per_layer = (len(kernels_only) - 4) // args.layers
        first = 2 + per_layer * min(2, args.layers - 1)           # a layer in the middle of the model
        before = kernels_only[first - 1].time_range.end
        print(f"step span {step[-1].time_range.end - step[0].time_range.start:.1f} us, {len(kernels_only)} kernels")
        for e in kernels_only[first: first + per_layer]:
            print(f"  ends {e.time_range.end - before:6.1f} us after the kernel before   {e.name[:70]}")
            before = e.time_range.end
        return 0
    if args.profile == "prefill":
        slot = engine.open_slot()
        prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        engine.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        torch.cuda.synchronize()
        print("profile run: one prefill of", PREFILL_TOKENS, "tokens")
        return 0

    # ---- prefill: one prompt of 2,048 tokens, logits at its last place
    prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(2 + 3):
        slot = engine.open_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close_slot(slot)
        if i >= 2:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    print("prefill runs (ms):", " ".join(f"{t:.2f}" for t in times), file=sys.stderr)
    flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}

    # ---- decode at batch 8, context 4,096: the headline
    with ClockSampler() as clocks:
        ms, launches = time_decode(engine, BATCH, CONTEXT, steps, warmup)
    value = BATCH / ms * 1e3
    step_bytes = nums["weight_bytes"] + BATCH * (CONTEXT - steps / 2) * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]}

    points, e2e, workloads = {}, None, {}
    if not args.quick:
        # ---- end to end through Engine.generate: host token lists in, host token lists out; directly after
        # `value`, as in the reference arm, whose two numbers come from one timed region
        # (as for ``value`` and for the reference arm: W untimed decode steps first, then K timed ones that end
        # at the benchmark context.  The stream runs one step ahead of its reader, so after the first token
        # and W more rows W + 1 steps have been launched and K are left.)
        new = steps + warmup + 2
        prompts = [torch.randint(0, cfg["vocab_size"], (CONTEXT - new,), generator=g).tolist() for _ in range(BATCH)]
        stream = engine.generate(prompts, new)
        for _ in range(1 + warmup):
            next(stream)                               # the prefill and the first token, then the warm-up steps
        torch.cuda.synchronize()
        begin = time.perf_counter()
        rows = sum(1 for _ in stream)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
        assert rows == steps + 1
        produced = steps
        batch = next(iter(b for b in engine.decoder.batches.values() if b.n == BATCH))
        e2e = {"value": round(BATCH * produced / elapsed, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(batch.h2d_bytes_per_step),
               "d2h_bytes_per_step": BATCH * 4 + 32}
        for name, n in (("decode_b1", 1), ("decode_b64", 64)):
            point_ms, _ = time_decode(engine, n, CONTEXT, max(8, steps // 4), warmup)
            points[name] = round(n / point_ms * 1e3, 1)
        # the benchmark configuration's other reading: prompts of 512 tokens, then the generated tokens
        for name, n in (("decode_b1_prompt512", 1), ("decode_b8_prompt512", BATCH), ("decode_b64_prompt512", 64)):
            point_ms, _ = time_decode(engine, n, PROMPT_OF_POINTS + steps + warmup + 1, steps, warmup)
            points[name] = round(n / point_ms * 1e3, 1)
        # the reference's own public workloads, measured as its harness measures them (bench/harness.py:26-30,
        # :81-110): a whole generate call by the wall clock, prefill included
        for name, batch, length, out_tokens in PUBLIC_WORKLOADS:
            workloads[name] = time_workload(engine, batch, length, out_tokens, cfg["vocab_size"], g)
        # last, because they make the cache anew: one sequence at 16,384 and at 32,768 tokens
        for name, context in (("decode_b1_context16k", 16384), ("decode_b1_context32k", 32768)):
            point_ms, _ = time_decode(long_engine(engine, context), 1, context, max(8, steps // 8), warmup)
            points[name] = round(1 / point_ms * 1e3, 1)

    line = {
        "metric": "decode tokens/s at batch 8 (Qwen3-4B sizes, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids, random cache content",
        "impl": "ours",
        "config": headline_config(args.layers),
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "workloads": workloads,
        "gpu_launches": int(launches * steps), "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
