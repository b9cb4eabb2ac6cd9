"""Command line: ``python -m starter_b200 <command>``.

The reference has no command line of its own for the engine; the options below use
its names where it has them (``model_path``, ``input_ids``, ``max_new_tokens``:
README.md:54-66).

  generate      --model-path DIR --input-ids "1,2,3;4,5" --max-new-tokens N
                [--temperature T] [--seed S] [--stop-token-ids 7,9] [--dtype bfloat16|float32]
                [--max-batch B]                 prints one JSON line per prompt
                instead of --input-ids: --prompt-lens 5,3 [--prompt-seed P] draws uniform random ids
  random-model  --config CONFIG.json --seed S --out DIR [--dtype float32|bfloat16]
                                                writes config.json and model.safetensors
  replay        --model DIR --dtype D --out DIR --max-tokens N      (bin/trace_run; steps on stdin)
"""

from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list:
    prompts = []
    for part in text.split(";"):
        part = part.strip()
        if part:
            prompts.append([int(t) for t in part.replace(" ", ",").split(",") if t != ""])
    return prompts


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="starter_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate from prompts given as token ids")
    gen.add_argument("--model-path", required=True, help="folder with config.json and safetensors")
    gen.add_argument("--input-ids", default=None,
                     help='token ids, prompts separated by ";": "1,2,3;4,5"; or @FILE with a JSON list of lists')
    gen.add_argument("--prompt-lens", default=None,
                     help="instead of --input-ids: comma-separated lengths of uniform random prompts")
    gen.add_argument("--prompt-seed", type=int, default=0, help="seed of the random prompts")
    gen.add_argument("--max-new-tokens", type=int, required=True)
    gen.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (default)")
    gen.add_argument("--seed", type=int, default=0, help="sampling seed")
    gen.add_argument("--stop-token-ids", default="", help="comma-separated ids that end a sequence")
    gen.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    gen.add_argument("--max-batch", type=int, default=64)

    rnd = sub.add_parser("random-model", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json of the architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])

    sub.add_parser("replay", help="trace replay (same as bin/trace_run)", add_help=False)

    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    args = parser.parse_args(argv)
    if args.command == "random-model":
        from .config import config_from_dict
        from .engine.runner import resolve_dtype
        from .weights import write_model_folder

        with open(args.config) as handle:
            config = config_from_dict(json.load(handle))
        write_model_folder(args.out, config, args.seed, resolve_dtype(args.dtype))
        print(json.dumps({"wrote": args.out, "seed": args.seed, "dtype": args.dtype}))
        return 0

    from .engine.entry import Engine

    if (args.input_ids is None) == (args.prompt_lens is None):
        parser.error("give exactly one of --input-ids and --prompt-lens")
    if args.prompt_lens is not None:
        import torch

        from .config import load_config

        vocab = load_config(args.model_path).vocab_size
        draw = torch.Generator().manual_seed(args.prompt_seed)
        prompts = [torch.randint(0, vocab, (int(n),), generator=draw).tolist()
                   for n in args.prompt_lens.split(",") if n.strip()]
    elif args.input_ids.startswith("@"):
        with open(args.input_ids[1:]) as handle:
            prompts = json.load(handle)
    else:
        prompts = _ids(args.input_ids)
    stops = [int(t) for t in args.stop_token_ids.split(",") if t.strip()]
    engine = Engine(args.model_path, dtype=args.dtype, max_batch=args.max_batch)
    results = engine.complete(prompts, args.max_new_tokens, temperature=args.temperature,
                              seed=args.seed, stop_token_ids=stops)
    for i, done in enumerate(results):
        print(json.dumps({"index": i, "tokens": done.tokens, "finish_reason": done.finish_reason}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
