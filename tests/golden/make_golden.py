"""Writes the golden files beside this script: logits of samplecatalina/mini-serve's own
model code (miniserve/model/qwen3.py, run on the CPU in float32) for two tiny random
models, the hashed sampling noise of its sampler (miniserve/engine/sampler.py:29-46) and a
continuation it samples at temperature 0.7 (:86-100), and checks that the tests' plain
implementation agrees with all of it.

    python tests/golden/make_golden.py --reference /path/to/mini-serve

The stored files hold only numbers that the reference produced (token ids in, logits
out), none of its code. ``tests/test_plain.py`` re-checks the plain implementation
against them without needing the reference.
"""

from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from tests.plain import qwen3_plain as plain  # noqa: E402

SAMPLED, TEMPERATURE, SAMPLE_SEED = 24, 0.7, 11  # the sampled continuation: tokens, temperature, seed

CASES = {
    "tiny_a": dict(raw=plain.tiny_config_a(), seed=0, ids_seed=1, length=33),
    "tiny_b": dict(raw=plain.tiny_config_b(), seed=7, ids_seed=2, length=40),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of samplecatalina/mini-serve")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    from miniserve.engine.sampler import Sampler, SamplingArgs, uniform_noise
    from miniserve.model.qwen3 import Qwen3Config, Qwen3ForCausalLM
    from miniserve.model.weights import load_config, load_weights

    for name, case in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            plain.write_random_model(tmp, case["raw"], case["seed"])
            g = torch.Generator().manual_seed(case["ids_seed"])
            ids = torch.randint(0, case["raw"]["vocab_size"], (case["length"],), generator=g)
            ref_model = Qwen3ForCausalLM(Qwen3Config.from_dict(load_config(Path(tmp))),
                                         load_weights(Path(tmp), device="cpu", dtype=torch.float32))
            n = len(ids)
            whole = ref_model.forward(ids, torch.arange(n), ref_model.new_cache(n), all_logits=True)
            # token by token through the reference's own cache, as a second view of the same numbers
            cache = ref_model.new_cache(n)
            step = torch.stack([ref_model.forward(ids[i:i + 1], torch.tensor([i]), cache) for i in range(n)])
            cfg, w = plain.read_config(tmp), plain.read_weights(tmp)
            ours = plain.all_logits(cfg, w, ids.tolist())
            # the sampler: its noise for a few (seed, counter) pairs, and 24 tokens it samples after a short prompt
            vocab = case["raw"]["vocab_size"]
            noise_keys = torch.tensor([[7, 40], [4000000000, 3], [0, 0], [123456789, 2303]], dtype=torch.int64)
            noise = uniform_noise(noise_keys[:, 0], noise_keys[:, 1], vocab)
            sampler = Sampler("cpu", vocab)
            seq = ids[:9].tolist()
            sampled = []
            for _ in range(SAMPLED):
                t = torch.tensor(seq)
                logits = ref_model.forward(t, torch.arange(len(seq)), ref_model.new_cache(len(seq)), all_logits=True)[-1:]
                args_ = SamplingArgs(torch.tensor([TEMPERATURE]), torch.tensor([1.0]), torch.tensor([SAMPLE_SEED]),
                                     torch.tensor([len(seq)]), False)
                sampled.append(int(sampler.sample(logits, args_)[0]))
                seq.append(sampled[-1])
            for row, (sd, ct) in zip(noise, noise_keys.tolist()):
                assert torch.equal(plain.uniform_noise(sd, ct, vocab), row), "plain noise differs from the reference's"
            mine = plain.generate(cfg, w, ids[:9].tolist(), SAMPLED, temperature=TEMPERATURE, seed=SAMPLE_SEED)
            assert mine == sampled, f"plain sampling differs from the reference's: {mine} != {sampled}"
        d_whole = (ours - whole).abs().max().item()
        d_step = (ours - step).abs().max().item()
        print(f"{name}: plain vs reference whole {d_whole:.3e}, vs reference token-by-token {d_step:.3e}, "
              f"reference whole vs token-by-token {(whole - step).abs().max().item():.3e}, "
              f"logit scale {whole.abs().max().item():.3f}")
        assert d_whole < 2e-5 and d_step < 2e-5, "plain implementation disagrees with the reference"
        save_file({"ids": ids.to(torch.int32), "logits": whole.contiguous(), "noise_keys": noise_keys,
                   "noise": noise.contiguous(), "sampled": torch.tensor(sampled, dtype=torch.int32)},
                  str(HERE / f"{name}.safetensors"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
