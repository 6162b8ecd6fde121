"""Command line: ``python -m flashdecode_cuda_b200 <command> ...``.

davidjoyme/flashdecode-cuda is driven by ``python -m <package>.<module>`` with
argparse options and ``FD_*`` environment variables (README.md:123-140); this
keeps that manner.  Commands:

``generate``        generate from prompts given as token ids (no tokenizer here)
``random-weights``  write a model folder (config.json, model.safetensors) from a
                    configuration and a seed
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _prompts(args) -> list:
    prompts = []
    for s in args.prompt_ids or []:
        prompts.append([int(t) for t in s.replace(" ", "").split(",") if t])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            data = json.load(f)
        prompts += [[int(t) for t in p] for p in data]
    if not prompts:
        raise SystemExit("give --prompt-ids 1,2,3 (repeatable) or --prompt-file FILE (JSON list of id lists)")
    return prompts


def cmd_generate(args) -> int:
    import flashdecode_cuda_b200 as fd
    if args.model:
        engine = fd.load(args.model, device=args.device, dtype=args.dtype)
    else:
        engine = fd.load(args.random, device=args.device, dtype=args.dtype, seed=args.seed)
    print(engine.config.summary(), file=sys.stderr)
    prompts = _prompts(args)
    stop = [int(t) for t in args.stop_ids.split(",")] if args.stop_ids else \
        (engine.config.stop_token_ids() if args.model else [])
    max_batch = args.max_batch or min(len(prompts), 64)
    longest = args.max_context or max(len(p) for p in prompts) + args.max_new_tokens
    cache = engine.new_paged_cache(max_batch, longest, args.block_size)
    t0 = time.time()
    results = engine.generate(prompts, args.max_new_tokens, cache, temperature=args.temperature,
                              seed=args.sample_seed, stop_token_ids=stop, max_batch=max_batch)
    dt = time.time() - t0
    n = sum(len(r.tokens) for r in results)
    for r in results:
        print(json.dumps({"request": r.request_id, "tokens": r.tokens, "finish_reason": r.finish_reason}))
    print(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s, prompts included in the time)", file=sys.stderr)
    return 0


def cmd_random_weights(args) -> int:
    import flashdecode_cuda_b200 as fd
    folder = fd.write_random_model(args.out, args.config, args.seed, args.dtype, qkv_bias=not args.no_qkv_bias)
    print(folder)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m flashdecode_cuda_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens from prompts of token ids")
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="model folder (config.json + model.safetensors)")
    src.add_argument("--random", metavar="PRESET", help="a preset name or config.json; weights drawn from --seed")
    g.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids; repeat for several prompts")
    g.add_argument("--prompt-file", help="JSON file: list of lists of token ids")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    g.add_argument("--sample-seed", type=int, default=0)
    g.add_argument("--stop-ids", default="", help="comma-separated stop token ids (default: eos_token_id of a loaded model)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    g.add_argument("--block-size", type=int, default=64, help="tokens per cache block")
    g.add_argument("--max-batch", type=int, default=0, help="sequences that run together (default: all, up to 64)")
    g.add_argument("--max-context", type=int, default=0, help="longest sequence the cache is sized for")
    g.add_argument("--device", default="cuda")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random-weights", help="write a random-weights model folder")
    r.add_argument("--config", required=True, help="preset name, config.json or model folder")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    r.add_argument("--no-qkv-bias", action="store_true", help="leave the q/k/v biases out")
    r.set_defaults(fn=cmd_random_weights)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
