"""Top-k and top-p through the entry point (the reference's host route: softmax on the device, filter and draw on
the host): every drawn token lies inside the set that the plain implementation's logits allow, a request's tokens
follow from its seed alone, and the captured decode step and the launched one draw the same tokens."""
import numpy as np
import pytest
import torch

import tiny
from plain.qwen3_plain import forward_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return tiny.make_folder(tmp_path_factory.mktemp("filters"), "B", torch.float32)


def _engine(folder, **kw):
    from prelude_b200 import Engine
    args = dict(dtype="f32", device="cuda:0", page_size=8, num_pages=64, max_running_requests=8)
    args.update(kw)
    return Engine(folder, **args)


def _allowed(logits, temperature, top_k, top_p, slack=1e-3):
    """Tokens that the filters may leave, from float64 logits, with a little slack at the edges.  As the sampler
    (and the reference) does it: the softmax over the whole vocabulary; top-k zeroes all but the k largest and
    does not renormalise; top-p then walks what is left from the largest down and stops once the mass before a
    token has reached top_p (skipped when what is left weighs less than top_p)."""
    z = logits.double().numpy() / temperature
    order = np.argsort(-z, kind="stable")
    p = np.exp(z - z.max())
    p /= p.sum()
    keep = np.ones(z.shape[0], dtype=bool)
    if top_k:
        keep &= z >= z[order[top_k - 1]] - slack
        p = np.where(keep, p, 0.0)
    if top_p < 1.0 and top_p < p.sum() + slack:
        before = np.cumsum(p[order]) - p[order]
        inside = np.zeros_like(keep)
        inside[order[before < top_p + slack]] = True
        keep &= inside
    return keep


@pytest.mark.parametrize("top_k,top_p", [(3, 1.0), (None, 0.6), (6, 0.8)])
def test_drawn_tokens_lie_inside_the_filtered_set(folder, top_k, top_p):
    cfg, w = tiny.PARAMS["B"][0], tiny.read_weights(folder)
    prompts = [tiny.random_ids(n, cfg["vocab_size"], 90 + n) for n in (5, 19, 33)]
    T, new = 1.3, 10
    outs = {}
    for graphs in (True, False):
        eng = _engine(folder, cuda_graph=graphs)
        res = eng.generate(prompts, temperature=T, top_k=top_k, top_p=top_p, seed=11, max_new_tokens=new, ignore_eos=True)
        outs[graphs] = [r.token_ids for r in res]
        # alone: the same tokens as in the batch
        assert eng.generate(prompts[1], temperature=T, top_k=top_k, top_p=top_p, seed=11, max_new_tokens=new,
                            ignore_eos=True).token_ids == outs[graphs][1]
        eng.cache.check()
    assert outs[True] == outs[False]
    distinct = set()
    for prompt, toks in zip(prompts, outs[True]):
        assert len(toks) == new
        logits = forward_logits(cfg, w, prompt + toks)
        for i, tok in enumerate(toks):
            allowed = _allowed(logits[len(prompt) + i - 1], T, top_k, top_p)
            assert allowed[tok], f"token {tok} at step {i} is outside the filtered set of {int(allowed.sum())} tokens"
            distinct.add(int(allowed.sum()))
    assert max(distinct) > 1                                  # the filters left a choice somewhere, not greedy in disguise
    # another seed, other tokens
    eng = _engine(folder)
    other = eng.generate(prompts, temperature=T, top_k=top_k, top_p=top_p, seed=12, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in other] != outs[True]


def _philox_uniform(seed, counter):
    """Philox4x32-10 restated in Python (Salmon et al. 2011): the number the sampler draws for (seed, counter)."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (c[0] >> 8) / 16777216.0


def _check_inverse_cdf(cfg, w, prompt, tokens, temperature, seed):
    """Token i of a request is the first index whose cumulative probability, in index order, exceeds
    philox(seed, i): over the plain implementation's softmax in float64, teacher-forced on the engine's tokens.
    Where the draw lands within rounding of a boundary, the neighbour is accepted."""
    logits = forward_logits(cfg, w, prompt + tokens, dtype=torch.float64)
    exact = 0
    for i, tok in enumerate(tokens):
        row = logits[len(prompt) - 1 + i]
        p = torch.exp((row - row.max()) / temperature)
        cum = torch.cumsum(p, 0)
        total = float(cum[-1])
        target = _philox_uniform(seed, i) * total
        want = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64), right=True))
        lo = float(cum[tok - 1]) if tok > 0 else 0.0
        hi = float(cum[tok])
        assert tok == want or abs(target - lo) < 1e-4 * total or abs(target - hi) < 1e-4 * total, \
            f"token {i}: drew {tok}, the seed's draw {target / total:.6f} falls on {want}"
        exact += tok == want
    return exact


@pytest.mark.parametrize("mode", ["launched", "graphs", "bursts", "preempted"])
def test_a_sampled_token_is_the_draw_of_its_seed_and_its_count(folder, mode):
    """Seed and count reach the kernel as they should through launched steps, captured steps, queued runs of
    captured steps, and across a preemption (the count goes on from the tokens already generated)."""
    cfg, w = tiny.PARAMS["B"][0], tiny.read_weights(folder)
    prompts = [tiny.random_ids(n, cfg["vocab_size"], 300 + n) for n in (6, 21, 11, 14)]
    seeds = [11, 2**40 + 5, 7, 11]
    T, new = 0.9, 18
    from prelude_b200 import SamplingParams
    sp = [SamplingParams(temperature=T, seed=s, max_new_tokens=new, ignore_eos=True) for s in seeds]
    kw = {"launched": dict(cuda_graph=False), "graphs": dict(decode_burst=1), "bursts": dict(decode_burst=6),
          "preempted": dict(decode_burst=1, num_pages=11, decode_reservation_cap=1)}[mode]
    eng = _engine(folder, **kw)
    res = eng.generate(prompts, sp)
    assert all(len(r.token_ids) == new for r in res)
    if mode == "preempted":
        assert sum(r.preemptions for r in res) >= 1
    if mode in ("graphs", "bursts"):
        assert eng.stats().graph_steps > 0
    exact = sum(_check_inverse_cdf(cfg, w, p, r.token_ids, T, s) for p, r, s in zip(prompts, res, seeds))
    assert exact >= len(prompts) * new - 2                     # boundary cases are rare
    eng.cache.check()
    assert eng.cache.used_pages() == 0
