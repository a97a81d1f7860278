"""Generates tests/golden/*.npz: logits and greedy tokens of the CPU oracle (oracle/rai_cpu.py) on the
tiny configurations of rai_b200.configs.TINY with seeded synthetic weights.

The reference itself cannot be built or run in this environment (no Rust toolchain), so these are
outputs of the restatement, not of rai: they pin the oracle against accidental change and give the
GPU tests a fixed target.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

import rai_cpu  # noqa: E402
import util  # noqa: E402
from rai_b200 import configs, synth  # noqa: E402

BATCH, PROMPT, STEPS = 2, 12, 6


def main():
    torch.set_num_threads(1)
    for i, name in enumerate(sorted(configs.TINY)):
        cfg = configs.get(name)
        seed = 4321 + i
        w = synth.weights(cfg, seed)
        model = util.build_oracle(cfg, w)
        prompt = synth.prompt(cfg, BATCH, PROMPT, seed)
        toks, logits = rai_cpu.greedy_generate(model, torch.from_numpy(prompt.astype(np.int64)), STEPS, True)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), seed=seed, prompt=prompt,
                            tokens=toks.numpy().astype(np.int64), logits=logits.numpy().astype(np.float32))
        print(name, "tokens", toks.tolist())


if __name__ == "__main__":
    main()
