"""Command-line options shared by every program that builds an engine.

Names, defaults and meanings follow miniserve/engine/cli.py:12-73 wherever this engine has the
same knob. Options of the reference that select between implementations this engine has only
one of are accepted with their single valid value, so that a command line written for the
reference keeps working.
"""

from __future__ import annotations

import argparse


def add_engine_args(parser: argparse.ArgumentParser) -> None:
    g = parser.add_argument_group("engine")
    g.add_argument("--max-running", type=int, default=64, help="how many requests may be admitted at the same time")
    g.add_argument("--max-prefill-tokens", type=int, default=8192,
                   help="without chunking (--chunked-prefill-size 0): the most prompt tokens one step takes")
    g.add_argument("--kv-pool-tokens", type=int, default=None,
                   help="size of the key/value cache in tokens, cut down to whole pages; unset: what the device has left")
    g.add_argument("--page-size", type=int, default=16, help="tokens in one cache page; a power of two")
    g.add_argument("--seed", type=int, default=0, help="where requests without a seed of their own get theirs from")
    g.add_argument("--chunked-prefill-size", type=int, default=None,
                   help="token budget of a step: decoding requests first, the rest filled with portions of prompts; "
                        "0 runs every prompt whole, in steps without decoding (default: 2048)")
    g.add_argument("--disable-cuda-graph", action="store_true", help="launch the kernels of every step one by one")
    g.add_argument("--disable-step-graphs", action="store_true",
                   help="keep the graphs of decode steps, launch prompt and mixed steps one kernel at a time")
    g.add_argument("--cuda-graph-max-bs", type=int, default=None,
                   help="decode steps up to this many requests replay a captured graph, padded to the next power of two "
                        "(from 16 on also the size halfway to it) or to this number (default: --max-running)")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: the serving kernels; float32: the whole model in true 32-bit")
    g.add_argument("--disable-overlap", action="store_true",
                   help="wait for a step's tokens before planning the next one (the host then idles while the GPU works)")
    g.add_argument("--poison-on-free", action="store_true",
                   help="debugging: fill the pages a request gives back with NaN, so that a stale read shows")
    # options of miniserve/engine/cli.py that choose between implementations of which this engine has one:
    # taken, with their single value, so that a command line written for that engine still parses
    g.add_argument("--attention", choices=["paged"], default="paged", help="the cache is always paged here")
    g.add_argument("--schedule-policy", choices=["fcfs", "sjf"], default="fcfs",
                   help="fcfs: waiting requests are tried in arrival order and the newest admitted one is preempted; sjf: least "
                        "remaining work first, most remaining work preempted (the reference's third policy, cache, orders by a "
                        "prefix cache, which is not here)")
    g.add_argument("--block-backend", choices=["cpp"], default="cpp", help="page bookkeeping is always the C++ one here")
    g.add_argument("--disable-radix", action="store_true", help="accepted and ignored: there is no prefix cache here")
    g.add_argument("--fused-ops", action="store_true", help="accepted and ignored: the fused kernels are the only ones here")
    g.add_argument("--attn-workspace-mb", type=int, default=None,
                   help="accepted and ignored: the attention kernels' scratch memory is sized by the engine")


def engine_kwargs(args: argparse.Namespace) -> dict:
    return dict(
        max_running=args.max_running,
        max_prefill_tokens=args.max_prefill_tokens,
        kv_pool_tokens=args.kv_pool_tokens,
        page_size=args.page_size,
        seed=args.seed,
        chunked_prefill_size=args.chunked_prefill_size,
        cuda_graph=not args.disable_cuda_graph,
        step_graphs=not args.disable_step_graphs,
        cuda_graph_max_bs=args.cuda_graph_max_bs,
        overlap=not args.disable_overlap,
        poison_on_free=args.poison_on_free,
        schedule_policy=args.schedule_policy,
    )


def add_model_args(parser: argparse.ArgumentParser) -> None:
    g = parser.add_argument_group("model")
    g.add_argument("--model", default=None, help="a model folder: config.json and safetensors files")
    g.add_argument("--random", default=None, metavar="PRESET",
                   help="no folder: a model of these sizes with random weights (tiny-a, tiny-b, 0.6b, 1.7b, 8b, 32b)")
    g.add_argument("--weights-seed", type=int, default=0, help="the random weights are drawn from this seed")
