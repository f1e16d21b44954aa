"""Offline stress run: many requests of random length at once, run to completion.

Checks that the engine neither stalls nor loses pages under cache pressure and reports how
often requests were preempted; it measures no speed. Options as in
miniserve/tools/stress.py:27-84.

    python -m miniserve_b200.tools.stress --random tiny-b --num-requests 64 --kv-pool-tokens 2048
"""

from __future__ import annotations

import argparse
import json
import random
import sys

from ..engine.cli import add_engine_args, add_model_args, engine_kwargs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    add_model_args(ap)
    add_engine_args(ap)
    ap.add_argument("--num-requests", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, nargs=2, default=[4, 1024], metavar=("MIN", "MAX"))
    ap.add_argument("--max-new-tokens", type=int, nargs=2, default=[1, 256], metavar=("MIN", "MAX"))
    ap.add_argument("--workload-seed", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--capture-graphs-at-start", action="store_true",
                    help="capture the decode graphs before the clock starts (else each at its first use, inside the timed run)")
    ap.add_argument("--max-steps", type=int, default=1_000_000, help="fail if not done after this many steps")
    args = ap.parse_args(argv)

    from ..engine import LLM, RequestState, SamplingParams

    llm = LLM(args.model, random=args.random, weights_seed=args.weights_seed, dtype=args.dtype, **engine_kwargs(args))
    eng = llm.engine
    if args.capture_graphs_at_start:
        eng.capture_graphs(("greedy",) if args.temperature == 0 else ("temperature", "top_p") if args.top_p < 1 else ("temperature",))
    vocab = llm.model.spec.vocab_size
    rng = random.Random(args.workload_seed)
    reqs = []
    for _ in range(args.num_requests):
        prompt = [rng.randrange(vocab) for _ in range(rng.randint(*args.prompt_len))]
        params = SamplingParams(rng.randint(*args.max_new_tokens), frozenset(), args.temperature, args.top_p)
        reqs.append(eng.add_request(prompt, params))
    import time

    import torch

    steps = max_decode_batch = max_used = 0
    phases = {"prefill": 0, "mixed": 0, "decode": 0}
    torch.cuda.synchronize()
    began = time.perf_counter()
    while eng.has_unfinished:
        if steps >= args.max_steps:
            print(f"not finished after {steps} steps", file=sys.stderr)
            return 1
        plan = eng.step()
        steps += 1
        if plan is not None:
            phases[plan.phase] += 1
            if plan.phase != "prefill":
                max_decode_batch = max(max_decode_batch, plan.num_decode)
        max_used = max(max_used, max(g.allocator.num_used for g in eng.cache.groups))
        eng.cache.check_invariants()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    report = dict(
        engine=engine_kwargs(args), num_requests=len(reqs), seconds=round(seconds, 3), steps_by_phase=phases,
        tokens_per_second=round(sum(len(r.prompt_ids) + len(r.output_ids) for r in reqs) / seconds, 1),
        prompt_tokens=sum(len(r.prompt_ids) for r in reqs), output_tokens=sum(len(r.output_ids) for r in reqs),
        steps=steps, max_decode_batch=max_decode_batch, max_pages_used=max_used, pool_pages=eng.cache.num_pages,
        preemptions=eng.scheduler.num_preemptions, preempted_requests=sum(r.num_preemptions > 0 for r in reqs),
        all_finished=all(r.state is RequestState.FINISHED for r in reqs), pages_returned=eng.cache.is_idle(),
    )
    print(json.dumps(report, indent=2))
    return 0 if report["all_finished"] and report["pages_returned"] else 1


if __name__ == "__main__":
    sys.exit(main())
