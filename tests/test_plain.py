"""The plain implementation checked against independent restatements of its
parts and against its committed outputs (no GPU)."""
import importlib.util
import json
import math
import os

import pytest
import torch

import tiny
from plain import qwen3_plain as plain
from prelude_b200.weights.random_init import random_tensors

HERE = os.path.dirname(os.path.abspath(__file__))


def test_committed_outputs_still_hold():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(HERE, "golden", "plain_tiny.json")) as f:
        want = json.load(f)
    got = mod.compute()
    for which in want:
        assert got[which]["ids"] == want[which]["ids"] and got[which]["greedy"] == want[which]["greedy"]
        assert got[which]["last_logits_head"] == pytest.approx(want[which]["last_logits_head"], abs=1e-8)
        assert got[which]["sum_abs"] == pytest.approx(want[which]["sum_abs"], rel=1e-9)


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = plain.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]]))


def test_rope_tables_and_rotation():
    cos, sin = plain.rope_tables(8, 5, 10000.0)
    assert cos.shape == (5, 4) and torch.allclose(cos[0], torch.ones(4)) and torch.allclose(sin[0], torch.zeros(4))
    assert float(cos[3, 1]) == pytest.approx(math.cos(3 * 10000.0 ** (-2 / 8)), abs=1e-6)
    # rotation keeps the length of each pair, and q.k depends on the distance only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    cos, sin = plain.rope_tables(8, 40, 10000.0, torch.float64)
    q, k = q.double(), k.double()

    def rot(x, p):
        return plain.apply_rope(x, cos[p:p + 1], sin[p:p + 1])
    assert torch.allclose(rot(q, 7).norm(), q.norm())
    d1 = (rot(q, 9) * rot(k, 4)).sum()
    d2 = (rot(q, 30) * rot(k, 25)).sum()
    assert float(d1) == pytest.approx(float(d2), abs=1e-5)    # angles are float32 by definition
    # pairs are (j, j + D/2)
    e = torch.zeros(1, 1, 8, dtype=torch.float64)
    e[0, 0, 1] = 1.0
    out = rot(e, 3)[0, 0]
    assert set(torch.nonzero(out.abs() > 1e-12).flatten().tolist()) == {1, 5}


def _attention_loops(q, k, v, scale, window=None):
    L, nH, D = q.shape
    g = nH // k.shape[1]
    out = torch.zeros_like(q)
    for i in range(L):
        for h in range(nH):
            lo = 0 if window is None else max(0, i - window + 1)
            s = torch.tensor([float(q[i, h] @ k[j, h // g]) * scale for j in range(lo, i + 1)], dtype=q.dtype)
            p = torch.softmax(s, 0)
            out[i, h] = sum(p[n] * v[lo + n, h // g] for n in range(len(p)))
    return out


@pytest.mark.parametrize("window", [None, 3])
def test_attention_against_loops(window):
    torch.manual_seed(0)
    q, k, v = torch.randn(7, 6, 8).double(), torch.randn(7, 2, 8).double(), torch.randn(7, 2, 8).double()
    got = plain.causal_attention(q, k, v, 0.3, window)
    assert torch.allclose(got, _attention_loops(q, k, v, 0.3, window), atol=1e-12)


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_logits_do_not_look_ahead_and_head_is_tied_or_not(which):
    cfg, init, _ = tiny.PARAMS[which]
    w = random_tensors(cfg, **init)
    ids = tiny.random_ids(10, cfg["vocab_size"], 5)
    full = plain.forward_logits(cfg, w, ids, torch.float64)
    assert full.shape == (10, cfg["vocab_size"])
    part = plain.forward_logits(cfg, w, ids[:6], torch.float64)
    assert torch.allclose(full[:6], part, atol=1e-12)
    changed = plain.forward_logits(cfg, w, ids[:6] + [(ids[6] + 1) % cfg["vocab_size"]] + ids[7:], torch.float64)
    assert torch.allclose(full[:6], changed[:6], atol=1e-12) and not torch.allclose(full[6:], changed[6:])
    assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])


def test_float32_is_close_to_float64():
    cfg, init, _ = tiny.PARAMS["B"]
    w = random_tensors(cfg, **init)
    ids = tiny.random_ids(40, cfg["vocab_size"], 6)
    a = plain.forward_logits(cfg, w, ids, torch.float32)
    b = plain.forward_logits(cfg, w, ids, torch.float64)
    assert float((a.double() - b).abs().max()) < 2e-5


def test_order_list_and_shared_keys():
    cfg, init, _ = tiny.PARAMS["A"]
    w = random_tensors(cfg, **init)
    ids = tiny.random_ids(9, cfg["vocab_size"], 7)
    default = plain.forward_logits(cfg, w, ids)
    assert torch.equal(default, plain.forward_logits(cfg, w, ids, order=[(0, None), (1, None)]))
    twice = plain.forward_logits(cfg, w, ids, order=[(0, None), (1, None), (0, None)])
    shared = plain.forward_logits(cfg, w, ids, order=[(0, None), (1, 0)])
    assert not torch.allclose(default, twice) and not torch.allclose(default, shared)


def test_greedy_takes_the_first_of_equal_logits():
    cfg = dict(tiny.TINY_A)
    w = {k: torch.zeros_like(v) for k, v in random_tensors(cfg).items()}
    assert plain.greedy_generate(cfg, w, [3, 4], 2) == [0, 0]
