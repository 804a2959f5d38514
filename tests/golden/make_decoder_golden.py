"""Writes tests/golden/qwen05b_q8_0_greedy.npz: the CPU oracle's greedy decode of the whole
Qwen2.5-0.5B-shaped Q8_0 decoder (random-init weights from the reference's PRNG, seed 23; a prompt of
128 uniform random ids, seed 29; 128 greedy tokens) with the margin between the two largest logits at
every step.  Run from the repository root: ``python tests/golden/make_decoder_golden.py`` (minutes of CPU,
about 5 GB of memory).  The GPU test rebuilds the same weights from the seed and compares token ids."""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))

import oracle  # noqa: E402
from neura_b200.qwen import QWEN25_05B_Q8  # noqa: E402
from oracle.decoder import OracleDecoder, synthetic_model  # noqa: E402

PROMPT, STEPS, SEED, PROMPT_SEED = 128, 128, 23, 29


def prompt_ids(config):
    return (oracle.Stream(PROMPT_SEED).uniform(PROMPT, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(1, PROMPT)


def main():
    config = QWEN25_05B_Q8
    began = time.time()
    packed, norms = synthetic_model(config, seed=SEED)
    print(f"weights drawn and packed in {time.time() - began:.1f} s", flush=True)
    prompts = prompt_ids(config)
    began = time.time()
    decoder = OracleDecoder(config, packed, norms, batch=1, capacity=PROMPT + STEPS, threads=os.cpu_count() or 1)
    tokens, margins = decoder.generate(prompts, STEPS)
    print(f"{PROMPT + STEPS - 1} steps in {time.time() - began:.1f} s; smallest margin {margins.min():.3e}", flush=True)
    out = os.path.join(os.path.dirname(__file__), "qwen05b_q8_0_greedy.npz")
    np.savez_compressed(out, prompt=prompts, tokens=tokens, margins=margins,
                        seeds=np.array([SEED, PROMPT_SEED], dtype=np.uint32))
    print("wrote", out)


if __name__ == "__main__":
    main()
