"""Offline stress run: many requests of random length, all submitted at once and run to the end.

It answers whether the engine gets through cache pressure (no stall, no page lost, everything
finished) and says how often it had to preempt; tokens per second are reported but it is no
benchmark. The workload options and the keys of the report are those of
miniserve/tools/stress.py:27-84, so that runs of the two engines can be laid side by side.

    python -m miniserve_b200.tools.stress --random tiny-b --num-requests 64 --kv-pool-tokens 2048
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time

from ..engine.cli import add_engine_args, add_model_args, engine_kwargs


class Watcher:
    """What a stress run notes after every step (``Engine.generate(on_step=...)``)."""

    def __init__(self):
        self.steps = 0
        self.by_phase = {"prefill": 0, "mixed": 0, "decode": 0}
        self.widest_decode = 0
        self.most_pages = 0

    def __call__(self, engine, plan) -> None:
        self.steps += 1
        if plan is not None:
            self.by_phase[plan.phase] += 1
            self.widest_decode = max(self.widest_decode, plan.num_decode)
        self.most_pages = max([self.most_pages] + [g.allocator.num_used for g in engine.cache.groups])
        engine.cache.check_invariants()


def workload(vocab: int, count: int, prompt_len, new_tokens, seed: int, temperature: float, top_p: float):
    from ..engine import SamplingParams

    rng = random.Random(seed)
    prompts, params = [], []
    for _ in range(count):
        prompts.append([rng.randrange(vocab) for _ in range(rng.randint(*prompt_len))])
        params.append(SamplingParams(rng.randint(*new_tokens), frozenset(), temperature, top_p))
    return prompts, params


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
                    help="capture every decode graph, and the step graphs of lone prompts, before the clock starts instead of at their first use")
    ap.add_argument("--max-steps", type=int, default=1_000_000, help="give up (exit code 1) after this many steps")
    args = ap.parse_args(argv)

    import torch

    from ..engine import LLM

    llm = LLM(args.model, random=args.random, weights_seed=args.weights_seed, dtype=args.dtype, **engine_kwargs(args))
    engine = llm.engine
    if args.capture_graphs_at_start:
        modes = ("greedy",) if args.temperature == 0 else ("temperature", "top_p") if args.top_p < 1 else ("temperature",)
        engine.capture_graphs(modes, context_lengths=(args.prompt_len[0], args.prompt_len[1] + args.max_new_tokens[1]),
                              prompt_tokens=args.prompt_len[1])
    prompts, params = workload(llm.model.spec.vocab_size, args.num_requests, args.prompt_len, args.max_new_tokens,
                               args.workload_seed, args.temperature, args.top_p)
    watch = Watcher()
    torch.cuda.synchronize()
    began = time.perf_counter()
    try:
        outputs = engine.generate(prompts, params, on_step=watch, max_steps=args.max_steps)
    except RuntimeError as e:
        print(e, file=sys.stderr)
        return 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    finished = all(len(o) == p.max_new_tokens for o, p in zip(outputs, params))  # no stop tokens are set
    prompt_tokens, output_tokens = sum(map(len, prompts)), sum(map(len, outputs))
    report = dict(
        engine=engine_kwargs(args), num_requests=len(prompts), seconds=round(seconds, 3), steps_by_phase=watch.by_phase,
        tokens_per_second=round((prompt_tokens + output_tokens) / seconds, 1),
        prompt_tokens=prompt_tokens, output_tokens=output_tokens,
        steps=watch.steps, max_decode_batch=watch.widest_decode, max_pages_used=watch.most_pages,
        pool_pages=engine.cache.num_pages, preemptions=engine.scheduler.num_preemptions,
        preempted_requests=engine.scheduler.num_preempted_requests,
        all_finished=finished, pages_returned=engine.cache.is_idle(),
        graphs_captured=dict(decode=len(engine.graphs._graphs) if engine.graphs is not None else 0,
                             steps=engine.step_fn.graphs.captures if getattr(engine.step_fn, "graphs", None) is not None else 0),
    )
    print(json.dumps(report, indent=2))
    return 0 if finished and report["pages_returned"] else 1


if __name__ == "__main__":
    sys.exit(main())
