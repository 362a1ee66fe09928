"""Command line: ``python -m rbitnet_b200 <verb>``.

The reference's own binary has no generation verb (its verbs are a model catalogue and
``serve``, crates/rbitnet-cli/src/main.rs:21-97); generation is reached through its
library call ``complete(prompt, max_tokens, temperature)`` and the environment variables
RBITNET_MODEL, RBITNET_TOKENIZER, RBITNET_TOY and RBITNET_TOY_SEED
(crates/bitnet-core/src/inference.rs:16-71).  The verbs here keep those names and
meanings: ``--max-tokens``, ``--temperature`` (<= 0 is greedy), ``--model`` defaulting to
$RBITNET_MODEL, ``--seed`` defaulting to $RBITNET_TOY_SEED or 42 for random weights.

  generate   token ids (or text, with tokenizer.json) in, generated ids (or text) out
  inspect    summary and tensor table of a model folder (in the manner of the
             reference's inspect_gguf example, crates/bitnet-core/examples/inspect_gguf.rs)
  random     write a model folder with seeded random weights for a config.json
  replay     trace replay (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path


def _add_engine_args(ap):
    ap.add_argument("--model", default=os.environ.get("RBITNET_MODEL"),
                    help="model folder (config.json, model.safetensors); default $RBITNET_MODEL")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--max-seq", type=int, default=None, help="longest sequence (default: the model's)")
    ap.add_argument("--cache-tokens", type=int, default=None, help="cache size in positions over all live sequences")
    ap.add_argument("--max-batch", type=int, default=64, help="most sequences generated together")


def _engine(args):
    from .engine import Engine
    if not args.model:
        raise SystemExit("no model: give --model DIR or set RBITNET_MODEL")
    kw = {"ops": args.ops} if getattr(args, "ops", None) is not None else {}
    return Engine.load_path(args.model, dtype=args.dtype, max_seq=args.max_seq, max_tokens=args.cache_tokens,
                            max_batch=args.max_batch, verbose=True, **kw)


def cmd_generate(args) -> int:
    eng = _engine(args)
    if args.prompt is not None:
        for text in args.prompt:
            print(eng.complete(text, args.max_tokens, args.temperature))
        return 0
    prompts = []
    for spec in args.prompt_ids or []:
        if os.path.isfile(spec):
            for line in Path(spec).read_text().splitlines():
                if line.strip():
                    prompts.append([int(t) for t in line.replace(",", " ").split()])
        else:
            prompts.append([int(t) for t in spec.replace(",", " ").split()])
    if not prompts:
        raise SystemExit("nothing to generate from: give --prompt TEXT or --prompt-ids '1 2 3' (or a file, one prompt a line)")
    stop = args.stop_id if args.stop_id else None
    results = eng.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature, seed=args.sample_seed,
                           stop_ids=stop)
    for r in results:
        print(json.dumps({"tokens": r.tokens, "finish_reason": r.finish_reason, "prompt_tokens": r.prompt_tokens}))
    return 0


def cmd_inspect(args) -> int:
    from .config import load_config, get_architecture
    from .weights import read_model_tensors, check_tensors
    cfg = load_config(args.model)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = read_model_tensors(args.model)
    n = sum(t.numel() for t in tensors.values())
    print(f"{cfg.architecture}: {len(spec.layers)} layers, width {spec.width}, vocabulary {spec.vocab_size}, "
          f"{len(tensors)} tensors, {n} parameters")
    for k, v in cfg.to_dict().items():
        print(f"  {k}: {v}")
    for name in sorted(tensors)[:args.max_names]:
        t = tensors[name]
        print(f"  {name}  {list(t.shape)}  {str(t.dtype).replace('torch.', '')}")
    check_tensors(spec.expected_shapes(), tensors, where=str(args.model), ignorable=spec.ignorable)
    print("tensors fit the model")
    return 0


def cmd_random(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(Path(args.config).read_text()))
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    out = write_random_model(args.out, cfg, args.seed, dtype=dt)
    print(f"wrote {out}/config.json and {out}/model.safetensors (seed {args.seed})")
    return 0


def main(argv=None, ops=None) -> int:
    """``ops``: a stand-in for the kernel layer (tests without a GPU); never given on the command line."""
    ap = argparse.ArgumentParser(prog="rbitnet_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="verb", required=True)
    g = sub.add_parser("generate", help="generate from token ids or text")
    _add_engine_args(g)
    g.add_argument("--prompt", action="append", help="text prompt (needs tokenizer.json); repeatable")
    g.add_argument("--prompt-ids", action="append", help="token ids '1 2 3', or a file with one prompt a line; repeatable")
    g.add_argument("--max-tokens", type=int, default=256, help="most new tokens per prompt (reference server default 256)")
    g.add_argument("--temperature", type=float, default=0.7, help="<= 0: greedy (reference server default 0.7)")
    g.add_argument("--sample-seed", type=int, default=0, help="seed of the sampling draws")
    g.add_argument("--stop-id", type=int, action="append", help="stop token id (default: config.json's eos_token_id)")
    g.set_defaults(fn=cmd_generate)
    i = sub.add_parser("inspect", help="summary and tensor table of a model folder")
    i.add_argument("model")
    i.add_argument("--max-names", type=int, default=20)
    i.set_defaults(fn=cmd_inspect)
    r = sub.add_parser("random", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=int(os.environ.get("RBITNET_TOY_SEED", "42")))
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.set_defaults(fn=cmd_random)
    p = sub.add_parser("replay", help="trace replay; arguments as bin/trace_run", add_help=False)
    p.set_defaults(fn=None)
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    args.ops = ops
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
