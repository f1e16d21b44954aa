"""Benchmark: decode tokens per second at a fixed batch and context, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of Qwen3-0.6B (28 layers, hidden 1024, 16 query heads, 8 kv heads,
head size 128, intermediate 3072, vocabulary 151,936, tied head) with random bfloat16 weights,
a batch of 8 requests whose context grows from 2,048 tokens on, one decode step per "step".
It prints ONE JSON line: ``value`` is decoded tokens per second timed on the device over exactly
K steps; ``e2e`` is the same through the Python entry point with host tokens in and out;
``prefill`` is one 2,048-token prompt; ``roofline`` is the decode step's bytes (every weight it
uses once, and the cache of the live requests) over its time against the measured copy
bandwidth; ``points`` holds decode at batch 1 and 64, at batch 8 behind 8,192 tokens and at batch 1 behind 32,768. This
engine runs on one GPU: for N > 1 it prints a line that says so and exits with 2.

``--config 8b`` and ``--config 32b`` run the two larger workloads instead (Qwen3-8B shapes: 32
requests with prompts of 128 to 4,096 tokens and 128 output tokens; Qwen3-32B shapes: 16 requests
with 8,192-token prompts and 128 output tokens, in a pool too small for all of them) through
``Engine.generate`` and print one line with tokens per second, the mean time of decode and of
mixed steps, their fraction of the measured peaks, and the number of preemptions.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONTEXT = 2048
DECODE_TOKENS = 256
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# --profile-range: the timed decode steps and the last timed prefill are bracketed by
# cudaProfilerStart/Stop, so that a profiler started with --profile-from-start off sees only them
PROFILE_RANGE = False


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))

            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return dict(hbm_gbs=flat["hbm_gbs"], bf16_tflops=flat["bf16_tflops"],
                            bf16_tflops_sustained=flat.get("bf16_tflops_sustained", flat["bf16_tflops"]),
                            source="measured")
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def qwen3_06b_config(layers: int | None) -> dict:
    from miniserve_b200.config import preset

    raw = preset("0.6b")
    if layers is not None:
        raw["num_hidden_layers"] = layers
    return raw


def flops_of_prefill(raw: dict, tokens: int) -> float:
    h, i, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    nq, nkv, d, layers = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["num_hidden_layers"]
    linear = 2.0 * tokens * ((nq + 2 * nkv) * d * h + nq * d * h + 3 * h * i) * layers
    attention = 4.0 * nq * d * (tokens * (tokens + 1) / 2) * layers  # causal half of QK^T and PV
    head = 2.0 * v * h  # one row of logits
    return linear + attention + head


class DecodeBench:
    """Holds B requests at a given context and steps them with synthetic next tokens."""

    def __init__(self, engine, batch: int, context: int, seed: int = 0):
        from miniserve_b200.engine.step import StepRow

        self.engine, self.batch, self.StepRow = engine, batch, StepRow
        self.rng = random.Random(seed)
        self.vocab = engine.model.spec.vocab_size
        self.caches = [engine.cache.new_request() for _ in range(batch)]
        step = engine.step_fn
        # prompts are prefilled in portions of at most 2,048 tokens per step (ids uniform over the vocabulary)
        for rc in self.caches:
            done = 0
            while done < context:
                n = min(2048, context - done)
                step.run([StepRow(rc, [self.rng.randrange(self.vocab) for _ in range(n)], ())])
                done += n
        self.context = context

    def rows(self):
        return [self.StepRow(rc, [self.rng.randrange(self.vocab)], (0,)) for rc in self.caches]

    def step_device(self):
        """One decode step without reading anything back (sampled tokens stay on the device)."""
        eng = self.engine
        if eng.graphs is not None and eng.graphs.takes(self.batch):
            return eng.graphs.run(self.rows(), None)
        logits = eng.step_fn.run(self.rows())
        return eng.sampler.sample(logits)

    def release(self):
        for rc in self.caches:
            self.engine.cache.release(rc)
        self.caches = []


def time_decode(engine, batch: int, context: int, steps: int, warmup: int):
    """(ms per step, launches per step, mean context during the timed steps)"""
    import torch

    from miniserve_b200.ops import native

    bench = DecodeBench(engine, batch, context)
    for _ in range(max(warmup, 3)):
        bench.step_device()
    torch.cuda.synchronize()
    start_ctx = bench.caches[0].num_tokens
    launches0 = native.LAUNCHES[0] + (engine.graphs.replayed_launches if engine.graphs is not None else 0)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if PROFILE_RANGE:
        torch.cuda.profiler.start()
    t0.record()
    for _ in range(steps):
        bench.step_device()
    t1.record()
    torch.cuda.synchronize()
    if PROFILE_RANGE:
        torch.cuda.profiler.stop()
    ms = t0.elapsed_time(t1) / steps
    launches = native.LAUNCHES[0] + (engine.graphs.replayed_launches if engine.graphs is not None else 0) - launches0
    mean_ctx = start_ctx + (steps + 1) / 2
    engine.step_fn.check_status()
    bench.release()
    return ms, launches / steps, mean_ctx


def time_e2e(llm, batch: int, context: int, steps: int, warmup: int):
    """The same decode steps through the public entry point: LLM.generate on host token ids.
    Prompts of ``context`` tokens are prefilled first; the timed region is the K decode steps that
    follow (each copies the step's inputs from pinned host memory and reads the sampled tokens
    back). Returns (tokens per second, h2d bytes per step, d2h bytes per step)."""
    import torch

    from miniserve_b200.engine import SamplingParams

    eng = llm.engine
    rng = random.Random(1)
    vocab = llm.model.spec.vocab_size
    prompts = [[rng.randrange(vocab) for _ in range(context)] for _ in range(batch)]
    # room to spare: a request that finished inside the timed region would shrink the batch
    reqs = [eng.add_request(p, SamplingParams(max_new_tokens=steps + warmup + 64)) for p in prompts]
    while any(r.state.name in ("WAITING", "PREFILL") for r in reqs):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    h2d0 = eng.step_fn.h2d_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (eng.step_fn.h2d_bytes - h2d0) / steps
    for r in list(reqs):
        eng.abort(r.rid)
    return batch * steps / dt, h2d, (batch + 1) * 4


def time_prefill(engine, tokens: int, repeats: int = 5, warmup: int = 6):
    import torch

    from miniserve_b200.engine.step import StepRow

    rng = random.Random(2)
    vocab = engine.model.spec.vocab_size
    ids = [rng.randrange(vocab) for _ in range(tokens)]
    times = []
    for i in range(repeats + warmup):
        rc = engine.cache.new_request()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if PROFILE_RANGE and i == repeats + warmup - 1:
            torch.cuda.profiler.start()
        t0.record()
        engine.step_fn.run([StepRow(rc, ids, (tokens - 1,))])
        t1.record()
        torch.cuda.synchronize()
        if PROFILE_RANGE and i == repeats + warmup - 1:
            torch.cuda.profiler.stop()
        if i >= warmup:  # the host's first passes are slower and a prompt step is close to host-bound
            times.append(t0.elapsed_time(t1))
        engine.cache.release(rc)
    return statistics.median(times)


def run_ours(args) -> dict:
    import torch

    from miniserve_b200.engine import LLM

    peaks = load_peaks()
    full_layers = qwen3_06b_config(None)["num_hidden_layers"]
    raw = qwen3_06b_config(args.layers)
    pool_tokens = 64 * (CONTEXT + DECODE_TOKENS) + 4096
    llm = LLM(random=raw, weights_seed=0, dtype="bfloat16", kv_pool_tokens=pool_tokens, page_size=16,
              max_running=64, chunked_prefill_size=2048, cuda_graph=not args.no_graph)
    eng = llm.engine
    model = llm.model
    weight_bytes = model.weight_bytes()
    kv_bytes_per_token = eng.cache.bytes_per_token()

    if args.only == "prefill":
        pre_ms = time_prefill(eng, PREFILL_TOKENS, repeats=max(1, min(args.steps, 5)))
        return {"impl": "ours", "only": "prefill", "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1),
                                                                "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 4)}}
    sampler = ClockSampler()
    sampler.start()
    ms, launches, mean_ctx = time_decode(eng, args.batch, CONTEXT, args.steps, args.warmup)
    clocks = sampler.stop()
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    if args.only == "decode":
        return {"impl": "ours", "only": "decode", "value": round(value, 1), "ms_per_step": round(ms, 4),
                "batch": args.batch, "gpu_launches": int(round(launches * args.steps)), "clocks": clocks,
                "roofline_frac": round(achieved / peaks["hbm_gbs"], 4)}
    points = {}
    for b in (1, 64):
        pms, _, _ = time_decode(eng, b, CONTEXT, min(args.steps, 128), args.warmup)
        points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
    points[f"decode_b{args.batch}"] = round(value, 1)
    long_ms, _, _ = time_decode(eng, 8, 4 * CONTEXT, min(args.steps, 64), args.warmup)
    points[f"decode_b8_ctx{4 * CONTEXT}"] = round(8 * 1000.0 / long_ms, 1)
    far_ms, _, _ = time_decode(eng, 1, 16 * CONTEXT, min(args.steps, 32), args.warmup)  # one request far into its context
    points[f"decode_b1_ctx{16 * CONTEXT}"] = round(1000.0 / far_ms, 1)

    pre_ms = time_prefill(eng, PREFILL_TOKENS)
    pre_flops = flops_of_prefill(raw, PREFILL_TOKENS)
    e2e_value, h2d, d2h = time_e2e(llm, args.batch, CONTEXT, min(args.steps, 128), args.warmup)

    return {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B shapes, context 2048->2304)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (token ids uniform over the vocabulary, random-init weights)",
        "impl": "ours",
        "config": {
            "model": "Qwen3-0.6B shapes", "layers": raw["num_hidden_layers"], "layers_full_model": full_layers,
            "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "tied_head": raw["tie_word_embeddings"], "global_batch": args.batch, "seq_len": CONTEXT,
            "decode_tokens": DECODE_TOKENS, "page_size": 16, "kv_pool_tokens": pool_tokens,
            "cuda_graph": eng.graphs is not None, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (1.19 GB of weights and the KV cache are read every step)",
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 4),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "peak": "burst"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"],
                     "step_bytes": int(step_bytes)},
        "points": points,
        "clocks": clocks,
    }


WORKLOADS = {
    # the reference's serving workload at Qwen3-8B sizes: continuous batching with a 2,048-token chunk budget, prompts uniform in [128, 4096]
    "8b": dict(preset="8b", requests=32, prompt=(128, 4096), new_tokens=128, pool_pages=None),
    # its workload at Qwen3-32B sizes: 16 prompts of 8,192 tokens in a pool that admits nine of them (a prompt and one token
    # each) and has 20 pages to spare: their 128 decoded tokens need 72, so admission stops AND requests are preempted
    "32b": dict(preset="32b", requests=16, prompt=(8192, 8192), new_tokens=128, pool_pages=9 * 513 + 20),
}


def run_workload(args) -> dict:
    import torch

    from miniserve_b200.config import preset
    from miniserve_b200.engine import LLM, SamplingParams

    peaks = load_peaks()
    wl = WORKLOADS[args.config]
    raw = preset(wl["preset"])
    full_layers = raw["num_hidden_layers"]
    if args.layers is not None:
        raw["num_hidden_layers"] = args.layers
    rng = random.Random(0)
    prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(rng.randint(*wl["prompt"]))] for _ in range(wl["requests"])]
    need = sum(len(p) + wl["new_tokens"] for p in prompts)
    pool_tokens = wl["pool_pages"] * 16 if wl["pool_pages"] else need + 4096
    llm = LLM(random=raw, weights_seed=0, dtype="bfloat16", kv_pool_tokens=pool_tokens, page_size=16, max_running=64,
              chunked_prefill_size=2048)
    eng = llm.engine
    eng.capture_graphs(("greedy",), context_lengths=(wl["prompt"][0], wl["prompt"][1] + wl["new_tokens"]))
    weight_bytes, kv_per_token = llm.model.weight_bytes(), eng.cache.bytes_per_token()
    h, inter = raw["hidden_size"], raw["intermediate_size"]
    nq, nkv, d, layers = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["num_hidden_layers"]
    per_token_flops = 2.0 * ((nq + 2 * nkv) * d * h + nq * d * h + 3 * h * inter) * layers
    events, steps = [], []

    def on_step(engine, plan):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        events.append(ev)
        if plan is None:
            steps.append(None)
            return
        ctx = sum(r.start + r.count for r in plan.rows)
        # attention flops of the step: every new token against the keys before and with it
        att = sum(4.0 * nq * d * (r.count * r.start + r.count * (r.count + 1) / 2) for r in plan.rows) * layers
        steps.append((plan.phase, plan.num_tokens, len(plan.rows), ctx, att))

    sampler = ClockSampler()
    sampler.start()
    torch.cuda.synchronize()
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=wl["new_tokens"]), on_step=on_step)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    clocks = sampler.stop()
    # device time of a step: from the end of the step before it to its own end
    times, prev = [], first
    for ev in events:
        times.append(prev.elapsed_time(ev))
        prev = ev
    decode = [(ms, s) for ms, s in zip(times, steps) if s is not None and s[0] == "decode"]
    mixed = [(ms, s) for ms, s in zip(times, steps) if s is not None and s[0] != "decode" and s[1] >= 2040]
    out_tokens = sum(len(o) for o in outs)
    result = {
        "impl": "ours", "workload": f"Qwen3-{args.config.upper()} shapes, {wl['requests']} requests, prompts {wl['prompt'][0]}..{wl['prompt'][1]}, "
                                    f"{wl['new_tokens']} output tokens each, chunk budget 2048",
        "layers": layers, "layers_full_model": full_layers, "dtype": "bf16", "kv_pool_tokens": pool_tokens,
        "tokens_needed_at_once": need, "seconds": round(seconds, 3),
        "value": round((sum(map(len, prompts)) + out_tokens) / seconds, 1), "unit": "tokens/s (prompt + output)",
        "output_tokens_per_s": round(out_tokens / seconds, 1), "steps": len(times),
        "preemptions": eng.scheduler.num_preemptions, "preempted_requests": eng.scheduler.num_preempted_requests,
        "all_finished": all(len(o) == wl["new_tokens"] for o in outs), "pages_returned": eng.cache.is_idle(),
        "weight_bytes": weight_bytes, "clocks": clocks,
    }
    if decode:
        ms = statistics.mean(t for t, _ in decode)
        byts = statistics.mean(weight_bytes + s[3] * kv_per_token for _, s in decode)
        result["decode_steps"] = {"count": len(decode), "mean_ms": round(ms, 3), "mean_batch": round(statistics.mean(s[2] for _, s in decode), 1),
                                  "mean_bytes": int(byts), "achieved_gbs": round(byts / ms / 1e6, 1),
                                  "frac_of_hbm_peak": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4), "peaks": peaks["source"]}
    if mixed:
        ms = statistics.mean(t for t, _ in mixed)
        flops = statistics.mean(per_token_flops * s[1] + s[4] for _, s in mixed)
        result["full_chunk_steps"] = {"count": len(mixed), "mean_ms": round(ms, 3), "mean_tokens": round(statistics.mean(s[1] for _, s in mixed), 1),
                                      "achieved_tflops": round(flops / ms / 1e9, 1),
                                      "frac_of_bf16_peak": round(flops / ms / 1e9 / peaks["bf16_tflops_sustained"], 4),
                                      "peak": "sustained"}
    return result


def run_reference(args) -> dict:
    """The unmodified reference from baseline/_ref through its own Engine.generate."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "miniserve").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref/miniserve is not installed on this box"}
    sys.path.insert(0, str(ref))
    try:
        import torch
        from miniserve.engine.engine import Engine
        from miniserve.engine.request import SamplingParams
        from miniserve.model.qwen3 import Qwen3Config, Qwen3ForCausalLM
        from miniserve.model.weights import expected_shapes
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference does not import here: {type(e).__name__}: {e}"[:300]}
    raw = qwen3_06b_config(args.layers)
    try:
        gen = torch.Generator(device="cuda").manual_seed(0)
        weights = {}
        for name, shape in expected_shapes(raw).items():
            t = torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32)
            weights[name] = ((1 + 0.1 * t) if len(shape) == 1 else 0.02 * t).to(torch.bfloat16)
        if raw.get("tie_word_embeddings"):
            weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
        model = Qwen3ForCausalLM(Qwen3Config.from_dict(raw), weights)
        # the faster of the reference's two stock configurations: its fused FlashInfer operators (--fused-ops),
        # where they build and run on this box; otherwise its default operators, with the reason
        kw = dict(max_running=64, kv_pool_tokens=64 * (CONTEXT + DECODE_TOKENS) + 4096, radix=False, chunked_prefill_size=2048)
        operators = "fused (fused_ops=True)"
        try:
            eng = Engine(model, fused_ops=True, **kw)
            probe = eng.add_request([1, 2, 3], SamplingParams(max_new_tokens=2))
            while eng.has_unfinished:
                eng.step()
            del probe
        except Exception as e:  # noqa: BLE001
            operators = f"default (fused_ops=True failed: {type(e).__name__}: {e})"[:160]
            eng = Engine(model, **kw)
        rng = random.Random(1)
        prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(CONTEXT)] for _ in range(args.batch)]
        reqs = [eng.add_request(p, SamplingParams(max_new_tokens=args.steps + args.warmup + 64)) for p in prompts]
        while any(r.state.name in ("WAITING", "PREFILL") for r in reqs):
            eng.step()
        for _ in range(max(args.warmup, 3)):
            eng.step()
        torch.cuda.synchronize()
        sampler = ClockSampler()
        sampler.start()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        clocks = sampler.stop()
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference's engine failed here: {type(e).__name__}: {e}"[:300]}
    ms = dt * 1000.0 / args.steps
    return {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B shapes, context 2048->2304)", "impl": "reference",
        "value": round(args.batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (token ids uniform over the vocabulary, random-init weights)",
        "config": {"model": "Qwen3-0.6B shapes", "layers": raw["num_hidden_layers"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "engine": "miniserve Engine.step (paged, CUDA graphs, overlap), wall clock",
                   "operators": operators},
        "e2e": {"value": round(args.batch * 1000.0 / ms, 1), "unit": "tokens/s"},
        "clocks": clocks,
    }


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DECODE_TOKENS)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--no-graph", action="store_true", help="run decode steps without CUDA graphs")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--config", choices=["0.6b", "8b", "32b"], default="0.6b",
                    help="0.6b: the benchmark line; 8b, 32b: the larger workloads through Engine.generate (a line of their own)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="measure only the decode steps or only the prefill (for profiling); the line then lacks the other parts")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unavailable": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                              "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    global PROFILE_RANGE
    PROFILE_RANGE = args.profile_range
    if args.config != "0.6b" and args.impl == "ours":
        result = run_workload(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
