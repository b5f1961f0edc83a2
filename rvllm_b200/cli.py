"""The command line, in the manner of the reference's `rvllm cli` (src/main.rs:33-131):

    rvllm cli --model DIR --prompt "..." [--prompt "..."] --max-tokens N
              [--arrival-step S ...] [--block-size 16] [--num-blocks N]
              [--temperature T] [--top-p P] [--seed 42] [--debug]

Option names, meanings and defaults are the reference's: each `--prompt` is one
concurrent request; `--arrival-step`, one per prompt in order, is the engine step at
which that request becomes eligible; `--max-tokens` defaults to 20; temperature 0 is
greedy; one completion is printed per line in prompt order.  Added here: `--token-ids`
(prompts are lists of token ids, printed back as ids), `--dtype`, `--prefill-chunk`,
`--max-batched-tokens`, and the `random-model` command, which writes a model folder
with random weights from a config.json and a seed.  The reference's interactive loop,
chat formatting, terminal UI and server are outside this engine.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="rvllm", description="LFM2 inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    cli = sub.add_parser("cli", help="run prompts to completion and print the answers")
    cli.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    cli.add_argument("--tokenizer", default=None,
                     help="tokenizer.json (default: the one beside the model)")
    cli.add_argument("--device", default="cuda", help="cuda or cuda:N (there is no CPU path)")
    cli.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    cli.add_argument("--block-size", type=int, default=16, help="tokens per KV page")
    cli.add_argument("--num-blocks", type=int, default=None,
                     help="KV pages in the pool (default: room for every request)")
    cli.add_argument("--prompt", action="append", default=[],
                     help="one request per occurrence")
    cli.add_argument("--token-ids", action="store_true",
                     help="prompts are token ids separated by spaces or commas")
    cli.add_argument("--max-tokens", type=int, default=20)
    cli.add_argument("--arrival-step", type=int, action="append", default=[],
                     help="one per --prompt, in order: the step at which it arrives")
    cli.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    cli.add_argument("--top-p", type=float, default=1.0)
    cli.add_argument("--seed", type=int, default=42)
    cli.add_argument("--prefill-chunk", type=int, default=None,
                     help="longest prompt portion per step")
    cli.add_argument("--max-batched-tokens", type=int, default=8192,
                     help="token budget of a step")
    cli.add_argument("--max-running", type=int, default=None)
    cli.add_argument("--debug", action="store_true",
                     help="also print prompts, steps, page allocations and throughput")
    rm = sub.add_parser("random-model", help="write a model folder with random weights")
    rm.add_argument("--config", required=True, help="a config.json")
    rm.add_argument("--seed", type=int, default=0)
    rm.add_argument("--out", required=True, help="folder to write")
    return ap


def run_cli(args) -> int:
    if not args.prompt:
        print("rvllm cli: give at least one --prompt (the interactive loop is not part of "
              "this engine)", file=sys.stderr)
        return 2
    if args.device.startswith("cpu") or args.device == "metal":
        print(f"rvllm cli: device {args.device!r} is not available: this engine runs on "
              f"CUDA only", file=sys.stderr)
        return 2
    from .engine import GenerateOptions, Generator
    gen = Generator.load(args.model, args.tokenizer, args.device, args.dtype)
    prompts = [_ids(p) for p in args.prompt] if args.token_ids else list(args.prompt)
    opts = GenerateOptions(max_tokens=args.max_tokens, temperature=args.temperature,
                           top_p=args.top_p, seed=args.seed, block_size=args.block_size,
                           num_blocks=args.num_blocks, prefill_chunk=args.prefill_chunk,
                           max_batched_tokens=args.max_batched_tokens,
                           max_running=args.max_running)
    outs = gen.complete_batch(prompts, opts, args.arrival_step)
    for i, (p, o) in enumerate(zip(args.prompt, outs)):
        text = " ".join(str(t) for t in o) if args.token_ids else o
        if args.debug:
            print(f"[{i}] prompt: {p}")
            print(f"[{i}] completion: {text}")
        else:
            print(text)
    if args.debug:
        s = gen.last_result.stats
        rate = s.output_tokens / s.elapsed if s.elapsed > 0 else 0.0
        print(f"steps: {s.steps}  prefill tokens: {s.prefill_tokens}  decode tokens: "
              f"{s.decode_tokens}  preemptions: {s.preemptions}")
        print(f"page allocations: {s.page_allocs}  pages high water: {s.pages_high_water}")
        print(f"{s.output_tokens} tokens in {s.elapsed:.3f} s = {rate:.1f} tok/s")
    return 0


def run_random_model(args) -> int:
    from .config import config_from_dict
    from .weights import write_random_model
    with open(args.config) as f:
        cfg = config_from_dict(json.load(f), args.config)
    write_random_model(args.out, cfg, args.seed)
    print(args.out)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "cli":
        return run_cli(args)
    return run_random_model(args)


if __name__ == "__main__":
    sys.exit(main())
