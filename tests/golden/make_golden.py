"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation
on the tiny configurations, so that an accidental edit of the oracle shows.

The reference's own model code (Rust on a forked tensor crate, fetched from git)
cannot be built or imported here, so these numbers come from tests/plain/qwen3_plain.py
itself and rest on the reference's formulas, not on its output.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import torch  # noqa: E402

import tiny  # noqa: E402
from plain.qwen3_plain import forward_logits, greedy_generate  # noqa: E402
from prelude_b200.weights.random_init import random_tensors  # noqa: E402


def compute():
    out = {}
    for which in "ABC":
        cfg, init, _ = tiny.PARAMS[which]
        w = random_tensors(cfg, **init)
        ids = tiny.random_ids(12, cfg["vocab_size"], 100 + ord(which))
        logits = forward_logits(cfg, w, ids, torch.float64)
        out[which] = {"ids": ids, "last_logits_head": [round(float(v), 9) for v in logits[-1, :8]],
                      "sum_abs": round(float(logits.abs().sum()), 6),
                      "greedy": greedy_generate(cfg, w, ids[:5], 6, torch.float64)}
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(compute(), f, indent=1)
    print("wrote plain_tiny.json")
