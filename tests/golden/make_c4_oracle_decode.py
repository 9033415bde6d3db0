"""Records the CPU oracle's greedy decode of the full 1B-architecture model (26 layers, 512-token
seeded prompt, 256 steps): the token ids and, per step, the margin between the two largest logits.

    python tests/golden/make_c4_oracle_decode.py [weight_seed] [prompt_seed]   (≈ 6 minutes on 8 cores)

writes tests/golden/c4_oracle_decode.json. The GPU parity test compares the device's free-running
greedy ids with a live oracle run and pins that run to this record.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from onyxia_b200 import llm, models  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    seed = int(sys.argv[1]) if len(sys.argv) > 1 else 0
    prompt_seed = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    steps = 256
    cfg = models.config_gemma3_1b()
    module = models.build_decoder(cfg, seed=seed)
    ref.set_threads(os.cpu_count() or 1)
    s = llm.LlmSession(ref.RefBackend(), module, 1024)
    prompt = np.random.default_rng(prompt_seed).integers(0, cfg.vocab, 512).tolist()
    logits = s.prefill(prompt)
    tokens, margins = [], []
    for _ in range(steps):
        top2 = np.sort(logits)[-2:]
        margins.append(float(top2[1] - top2[0]))
        tokens.append(int(llm.sample_greedy(logits)))
        logits = s.decode(tokens[-1])
    out = {"config": cfg.name, "seed": seed, "prompt_seed": prompt_seed, "prompt_len": 512, "tokens": tokens, "margins": margins,
           "min_margin": min(margins)}
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "c4_oracle_decode.json"), "w") as f:
        json.dump(out, f)
    print("min margin", min(margins), "five smallest", sorted(margins)[:5])


if __name__ == "__main__":
    main()
