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
    g.add_argument("--max-running", type=int, default=64, help="max requests in the running batch")
    g.add_argument("--max-prefill-tokens", type=int, default=8192, help="token budget of one prefill batch")
    g.add_argument("--kv-pool-tokens", type=int, default=None,
                   help="exact KV pool size in tokens (rounded down to whole pages); "
                        "default: as large as GPU memory allows")
    g.add_argument("--page-size", type=int, default=16, help="tokens per KV page (a power of two)")
    g.add_argument("--seed", type=int, default=0, help="seeds sampling for requests that bring no seed of their own")
    g.add_argument("--chunked-prefill-size", type=int, default=None,
                   help="tokens per step, decodes included, with prefills cut into chunks batched with decodes; "
                        "0: whole prefills in prefill-only steps (default: 2048)")
    g.add_argument("--disable-cuda-graph", action="store_true", help="run decode steps eagerly (no CUDA Graphs)")
    g.add_argument("--cuda-graph-max-bs", type=int, default=None,
                   help="largest decode batch captured in a CUDA Graph (default: --max-running); "
                        "graphs are captured for powers of two below it and for it")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: the serving kernels; float32: the whole model in true 32-bit")
    # accepted for compatibility with the reference's command lines; one valid value each
    g.add_argument("--attention", choices=["paged"], default="paged", help="KV storage (only paged here)")
    g.add_argument("--schedule-policy", choices=["fcfs"], default="fcfs", help="admission order (only fcfs here)")
    g.add_argument("--block-backend", choices=["cpp"], default="cpp", help="block bookkeeping (C++ here)")
    g.add_argument("--disable-radix", action="store_true", help="no prefix cache (this engine has none)")
    g.add_argument("--disable-overlap", action="store_true",
                   help="read back each step's tokens before scheduling the next (no CPU-GPU overlap)")
    g.add_argument("--fused-ops", action="store_true", help="fused operators (this engine always uses its fused kernels)")


def engine_kwargs(args: argparse.Namespace) -> dict:
    return dict(
        max_running=args.max_running,
        max_prefill_tokens=args.max_prefill_tokens,
        kv_pool_tokens=args.kv_pool_tokens,
        page_size=args.page_size,
        seed=args.seed,
        chunked_prefill_size=args.chunked_prefill_size,
        cuda_graph=not args.disable_cuda_graph,
        cuda_graph_max_bs=args.cuda_graph_max_bs,
        overlap=not args.disable_overlap,
    )


def add_model_args(parser: argparse.ArgumentParser) -> None:
    g = parser.add_argument_group("model")
    g.add_argument("--model", default=None, help="folder with config.json and *.safetensors")
    g.add_argument("--random", default=None, metavar="PRESET",
                   help="instead of --model: random weights for a preset (tiny-a, tiny-b, 0.6b, 1.7b, 8b, 32b)")
    g.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
