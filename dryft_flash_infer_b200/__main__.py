"""Command line of the package: token ids in, token ids out (the engine has no tokenizer,
as the reference has none).

    python -m dryft_flash_infer_b200 generate --model DIR --prompt-ids prompts.json --max-new-tokens 32
    python -m dryft_flash_infer_b200 generate --model DIR --random-prompts 4:128 --max-new-tokens 16 --temperature 0.8 --seed 1
    python -m dryft_flash_infer_b200 generate --random-config config.json --random-prompts 8:512 --max-new-tokens 64
    python -m dryft_flash_infer_b200 random-model --config config.json --seed 0 --out DIR

``generate`` prints one JSON line per output step (the list that ``Engine.generate`` yields)
and a last line with tokens per second.  The reference engine is configured through
environment variables; the one that applies here keeps its name and meaning:
``DRYFT_GRAPH=on|off`` (capture the decode step, and short prompt steps, in CUDA graphs), also ``--cuda-graph``.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _generate(args) -> int:
    import torch

    from . import Engine

    options = {"dtype": args.dtype}
    if args.cuda_graph is not None:
        options["cuda_graph"] = args.cuda_graph == "on"
    if (args.model is None) == (args.random_config is None):
        raise SystemExit("give either --model DIR or --random-config CONFIG_JSON")
    if args.model is not None:
        engine = Engine(args.model, **options)
    else:
        # a model of random weights made on the device from a configuration file: no folder is written
        with open(args.random_config) as fh:
            engine = Engine(config=json.load(fh), random_weights=True, seed=args.seed, **options)
    if args.prompt_ids:
        with open(args.prompt_ids) as fh:
            prompts = json.load(fh)
        if not (isinstance(prompts, list) and all(isinstance(p, list) for p in prompts)):
            raise SystemExit("--prompt-ids must hold a JSON list of lists of token ids")
    elif args.random_prompts:
        batch, length = (int(v) for v in args.random_prompts.split(":"))
        g = torch.Generator().manual_seed(args.seed)
        prompts = torch.randint(0, engine.config.vocab_size, (batch, length), generator=g).tolist()
    else:
        raise SystemExit("give --prompt-ids FILE or --random-prompts BATCH:LENGTH")
    begin = time.perf_counter()
    steps = 0
    for row in engine.generate(prompts, args.max_new_tokens, temperature=args.temperature, seed=args.seed,
                               stop_token_ids=tuple(args.stop_token_id or ())):
        print(json.dumps(row), flush=True)
        steps += 1
    elapsed = time.perf_counter() - begin
    print(json.dumps({"steps": steps, "sequences": len(prompts), "seconds": round(elapsed, 4),
                      "tokens_per_second": round(len(prompts) * steps / elapsed, 1) if elapsed > 0 else None}))
    return 0


def _random_model(args) -> int:
    import torch

    from . import write_random_model
    from .config import config_from_dict

    with open(args.config) as fh:
        config = config_from_dict(json.load(fh))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    folder = write_random_model(config, args.seed, args.out, dtype)
    print(f"wrote {folder}/config.json and {folder}/model.safetensors")
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m dryft_flash_infer_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    gen = sub.add_parser("generate", help="continue prompts given as token ids")
    gen.add_argument("--model", help="folder with config.json and model.safetensors")
    gen.add_argument("--random-config", metavar="CONFIG_JSON",
                     help="instead of --model: a config.json of the architecture; the weights are random (--seed)")
    gen.add_argument("--prompt-ids", help="JSON file: a list of lists of token ids")
    gen.add_argument("--random-prompts", metavar="BATCH:LENGTH", help="seeded uniform-random prompts instead")
    gen.add_argument("--max-new-tokens", type=int, required=True)
    gen.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    gen.add_argument("--seed", type=int, default=0)
    gen.add_argument("--stop-token-id", type=int, action="append")
    gen.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    gen.add_argument("--cuda-graph", choices=["on", "off"], default=None, help="default: $DRYFT_GRAPH, else on")
    gen.set_defaults(run=_generate)
    rnd = sub.add_parser("random-model", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json of the architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    rnd.set_defaults(run=_random_model)
    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
