"""Time one kernel of the package on synthetic data of a given shape: the cases that the
summaries under ``profiles/`` were measured and captured with.

    python -m miniserve_b200.tools.kernel_bench attn_decode --batch 64 --context 2048
    python -m miniserve_b200.tools.kernel_bench attn_prefill --tokens 2048
    python -m miniserve_b200.tools.kernel_bench skinny --m 8 --n 4096 --k 1024
    python -m miniserve_b200.tools.kernel_bench sample --batch 8 --top-p 0.9

Each case rotates over enough copies of its inputs to exceed the L2 cache, captures one pass over
all copies in a CUDA graph, and reports the time per launch with the bytes or flops it implies.
``--launches N`` instead runs N plain launches (what a profiler attaches to).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
from types import SimpleNamespace

import torch

L2_BYTES = 160e6


def _paged(rows, page, nkv, d, seed, device):
    rng = random.Random(seed)
    need = [-(-(s + n) // page) for s, n in rows]
    order = list(range(sum(need) + 3))
    rng.shuffle(order)
    tables, at = [], 0
    for n in need:
        tables.append(order[at:at + n])
        at += n
    i32 = dict(dtype=torch.int32, device=device)
    k = torch.randn((len(order), nkv, page, d), device=device).bfloat16()
    v = torch.randn((len(order), nkv, page, d), device=device).bfloat16()
    indptr = [0]
    for t in tables:
        indptr.append(indptr[-1] + len(t))
    cu = [0]
    for _, n in rows:
        cu.append(cu[-1] + n)
    ctx = SimpleNamespace(
        num_rows=len(rows), num_tokens=cu[-1], cu_q=torch.tensor(cu, **i32),
        q_start=torch.tensor([s for s, _ in rows], **i32), kv_len=torch.tensor([s + n for s, n in rows], **i32),
        page_indptr=[torch.tensor(indptr, **i32)], page_indices=[torch.tensor([p for t in tables for p in t], **i32)],
        max_q_len=max(n for _, n in rows), max_kv_len=max(s + n for s, n in rows),
        decode_only=all(n == 1 for _, n in rows), host_q_start=[s for s, _ in rows], host_q_len=[n for _, n in rows],
        leading_single_rows=next((i for i, (_, n) in enumerate(rows) if n != 1), len(rows)), graph_bucket=0, scratch={}, step_cache={},
        sm_count=torch.cuda.get_device_properties(0).multi_processor_count, stream=0)
    return k, v, ctx


def _time(calls, copies, launches):
    """calls(i, stream) launches the kernel on input copy i."""
    s = torch.cuda.Stream()
    if launches:
        with torch.cuda.stream(s):
            for i in range(launches):
                calls(i % copies, s.cuda_stream)
        s.synchronize()
        return None
    with torch.cuda.stream(s):
        for i in range(copies):
            calls(i, s.cuda_stream)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(copies):
            calls(i, torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(7):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1000 / copies)
    return sorted(times)[len(times) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("kernel", choices=["attn_decode", "attn_prefill", "skinny", "add_rmsnorm", "gemm", "gate_up", "sample"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--prefix", type=int, default=0, help="attn_prefill: tokens already in the cache before the portion")
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--gemm", choices=["auto", "tcgen05", "library"], default="auto",
                    help="gemm, gate_up: this package's tcgen05 kernels, the vendor library, or the engine's choice")
    ap.add_argument("--vocab", type=int, default=151936, help="sample: tokens in a row of logits")
    ap.add_argument("--temperature", type=float, default=0.8, help="sample: 0 is greedy")
    ap.add_argument("--top-p", type=float, default=1.0, help="sample: below 1, the nucleus is found first")
    ap.add_argument("--launches", type=int, default=0, help="run this many plain launches and report nothing")
    args = ap.parse_args(argv)

    from .. import ops

    dev = torch.device("cuda:0")
    out = dict(kernel=args.kernel)
    if args.kernel in ("attn_decode", "attn_prefill"):
        nq, nkv, d = args.heads, args.kv_heads, args.head_dim
        if args.kernel == "attn_decode":
            rows = [(args.context, 1)] * args.batch
            byts = args.batch * (args.context + 1) * nkv * d * 2 * 2
            work = dict(bytes=byts)
        else:
            rows = [(args.prefix, args.tokens)]  # a portion of a prompt behind `prefix` cached tokens
            flops = 4.0 * nq * d * (args.tokens * (args.tokens + 1) / 2 + args.tokens * args.prefix)
            byts = (args.prefix + args.tokens) * nkv * d * 4
            work = dict(flops=flops)
        copies = max(2, int(L2_BYTES // byts) + 1)
        sets = [_paged(rows, args.page_size, nkv, d, i, dev) for i in range(copies)]
        q = torch.randn(sum(n for _, n in rows), nq, d, device=dev).bfloat16()
        o = torch.empty_like(q)

        def calls(i, stream):
            k, v, ctx = sets[i]
            ctx.stream = stream
            ops.attention(o, q, k, v, ctx, 0, d ** -0.5, None)
    elif args.kernel in ("gemm", "gate_up"):
        # gemm: x [m, k] times w [n, k]^T; gate_up: silu(x Wg^T) * (x Wu^T) with the stacked weight [2 n, k]
        ops.TC_GEMM = {"auto": "auto", "tcgen05": "1", "library": "0"}[args.gemm]
        rows = args.n * (2 if args.kernel == "gate_up" else 1)
        work = dict(flops=2.0 * args.m * rows * args.k)
        copies = max(2, int(L2_BYTES // (rows * args.k * 2)) + 1)
        ws = [(torch.randn(rows, args.k, device=dev) * args.k ** -0.5).bfloat16() for _ in range(copies)]
        x = torch.randn(args.m, args.k, device=dev).bfloat16()
        o = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        scratch = torch.empty(args.m, rows, device=dev, dtype=torch.bfloat16)

        def calls(i, stream):
            if args.kernel == "gemm":
                ops.linear(x, ws[i], out=o, stream=stream)
            else:
                ops.linear_silu_mul(x, ws[i], o, scratch=scratch, stream=stream)
    elif args.kernel == "sample":
        # --batch rows of float32 logits, each row with its own seed
        byts = args.batch * args.vocab * 4
        work = dict(bytes=byts)
        copies = max(2, min(16, int(L2_BYTES // byts) + 1))
        logits = [torch.randn(args.batch, args.vocab, device=dev) * 3 for _ in range(copies)]
        tokens = torch.empty(args.batch, dtype=torch.int32, device=dev)
        temp = torch.full((args.batch,), args.temperature, device=dev)
        top_p = torch.full((args.batch,), args.top_p, device=dev) if args.top_p < 1 else None
        seed = torch.arange(args.batch, dtype=torch.int64, device=dev)
        counter = torch.full((args.batch,), 5, dtype=torch.int64, device=dev)
        nucleus = torch.empty(args.batch * ops.nucleus_bytes(), dtype=torch.uint8, device=dev)

        def calls(i, stream):
            if args.temperature == 0:
                ops.sample(tokens, logits[i], stream=stream)
            else:
                ops.sample(tokens, logits[i], temperature=temp, top_p=top_p, seed=seed, counter=counter,
                           scratch=nucleus if top_p is not None else None, stream=stream)
    elif args.kernel == "skinny":
        byts = args.n * args.k * 2
        work = dict(bytes=byts)
        copies = max(2, int(L2_BYTES // byts) + 1)
        ws = [torch.randn(args.n, args.k, device=dev).bfloat16() for _ in range(copies)]
        x = torch.randn(args.m, args.k, device=dev).bfloat16()
        o = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)

        def calls(i, stream):
            ops.linear(x, ws[i], out=o, stream=stream)
    else:
        h = args.n
        byts = args.m * h * 10
        work = dict(bytes=byts)
        copies = 16
        res = torch.randn(args.m, h, device=dev)
        delta = torch.randn(args.m, h, device=dev).bfloat16()
        w = torch.ones(h, device=dev).bfloat16()
        o = torch.empty(args.m, h, device=dev, dtype=torch.bfloat16)

        def calls(i, stream):
            ops.add_rmsnorm(o, res, delta, w, 1e-6, stream=stream)
    us = _time(calls, copies, args.launches)
    if us is not None:
        out.update(us_per_launch=round(us, 2), copies=copies)
        if "bytes" in work:
            out.update(bytes=work["bytes"], tb_per_s=round(work["bytes"] / us / 1e6, 3))
        if "flops" in work:
            out.update(flops=work["flops"], tflops=round(work["flops"] / us / 1e6, 1))
    out.update({k: v for k, v in vars(args).items() if k != "kernel"})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
