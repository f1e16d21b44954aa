"""Generate tokens from token ids on the command line.

    python -m miniserve_b200.tools.generate --random tiny-a --prompt-ids 5,17,3 --max-new-tokens 8
    python -m miniserve_b200.tools.generate --model DIR --prompt-len 128 --num-prompts 4 --temperature 0.7

Token ids in, token ids out (as JSON): like the reference's engine, this path has no tokenizer
(miniserve/engine/engine.py:206-211).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time

from ..engine.cli import add_engine_args, add_model_args, engine_kwargs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    add_model_args(ap)
    add_engine_args(ap)
    ap.add_argument("--prompt-ids", action="append", default=None, metavar="ID,ID,...",
                    help="a prompt as comma-separated token ids (may be given several times)")
    ap.add_argument("--prompt-len", type=int, default=None, help="instead: random prompts of this many tokens")
    ap.add_argument("--num-prompts", type=int, default=1)
    ap.add_argument("--workload-seed", type=int, default=0)
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--stop-token-ids", default="", metavar="ID,ID,...")
    ap.add_argument("--capture-graphs-at-start", action="store_true",
                    help="capture the CUDA graphs that these requests will replay before the clock starts instead of at their first use")
    args = ap.parse_args(argv)

    from ..engine import LLM, SamplingParams

    llm = LLM(args.model, random=args.random, weights_seed=args.weights_seed, dtype=args.dtype, **engine_kwargs(args))
    vocab = llm.model.spec.vocab_size
    if args.prompt_ids:
        prompts = [[int(x) for x in p.split(",") if x.strip()] for p in args.prompt_ids]
    elif args.prompt_len:
        rng = random.Random(args.workload_seed)
        prompts = [[rng.randrange(vocab) for _ in range(args.prompt_len)] for _ in range(args.num_prompts)]
    else:
        ap.error("give --prompt-ids or --prompt-len")
    stop = frozenset(int(x) for x in args.stop_token_ids.split(",") if x.strip())
    params = SamplingParams(args.max_new_tokens, stop, args.temperature, args.top_p)
    if args.capture_graphs_at_start:
        modes = ("greedy",) if args.temperature == 0 else ("top_p",) if args.top_p < 1 else ("temperature",)
        longest = max(map(len, prompts))
        llm.engine.capture_graphs(modes, context_lengths=(min(map(len, prompts)), longest + args.max_new_tokens), prompt_tokens=longest)
    t0 = time.perf_counter()
    outputs = llm.generate(prompts, params)
    dt = time.perf_counter() - t0
    print(json.dumps(dict(outputs=outputs, seconds=round(dt, 4), steps=llm.engine.num_steps,
                          preemptions=llm.engine.scheduler.num_preemptions)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
