"""Writes tests/golden/plain_tiny.json: outputs of tests/plain_llama.py (float64)
for the two tiny configurations with seeded random weights.

The reference is Rust and cannot be compiled or imported in this environment,
so these numbers do not come from it; they pin the plain implementation, which
is written from the reference's formulas, against later change.
Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from plain_llama import plain_forward, plain_generate  # noqa: E402
from tiny import TINY_A, TINY_B, make_model  # noqa: E402

out = {}
for name, cfg, seed in (("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)):
    _, c, tensors = make_model(cfg, seed, torch.float32)
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg["vocab_size"], (17,), generator=g).tolist()
    logits = plain_forward(c, tensors, ids, torch.float64)
    out[name] = {"ids": ids, "last_logits_first8": logits[-1, :8].tolist(),
                 "greedy6": plain_generate(c, tensors, ids, 6)}
json.dump(out, open(os.path.join(HERE, "plain_tiny.json"), "w"), indent=1)
print("wrote", os.path.join(HERE, "plain_tiny.json"))
