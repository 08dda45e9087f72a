"""The host side of sampling: which sampler a request gets, the top-k and top-p filters after the reference
(crates/prelude-core/src/engine/sampling/logits_processor.rs:44-135), and the draw from what is left."""
import numpy as np
import pytest

from prelude_b200.sampling.sampler import draw, filter_top_k, filter_top_p, sampling_mode


def test_which_sampler():
    # postprocess.rs:18-38: a temperature below 1e-7 is greedy whatever else is set; top-k wins over top-p alone
    assert sampling_mode(0.0, 5, 0.5) == "greedy" and sampling_mode(5e-8, None, 1.0) == "greedy"
    assert sampling_mode(0.7, 5, 1.0) == "top_k_top_p" and sampling_mode(0.7, 5, 0.5) == "top_k_top_p"
    assert sampling_mode(0.7, None, 0.9) == "top_p" and sampling_mode(0.7, 0, 0.9) == "top_p"
    assert sampling_mode(0.7, None, 1.0) == "all" and sampling_mode(1e-7, 0, 1.0) == "all"


def _top_p_by_the_book(probs, top_p):
    """The reference's loop, word for word: walk the tokens from the most probable down; once the running sum has
    reached top_p, zero what follows."""
    order = sorted(range(len(probs)), key=lambda i: (-probs[i], i))
    out, cum = probs.copy(), 0.0
    for i in order:
        if cum >= top_p:
            out[i] = 0.0
        else:
            cum += float(probs[i])
    return out


def test_top_p_keeps_the_smallest_head_that_reaches_p():
    p = np.array([0.1, 0.4, 0.05, 0.3, 0.15], dtype=np.float32)
    assert filter_top_p(p, 0.5).tolist() == [0, p[1], 0, p[3], 0]            # 0.4 < 0.5: the next one is still kept
    assert filter_top_p(p, 0.4).tolist() == [0, p[1], 0, 0, 0]               # float32(0.4) is a hair above 0.4: reached
    assert filter_top_p(p, 0.39).tolist() == [0, p[1], 0, 0, 0]
    assert filter_top_p(p, 1.0).tolist() == p.tolist() and filter_top_p(p, 0.0).tolist() == [0] * 5
    assert p.tolist() == [np.float32(x) for x in (0.1, 0.4, 0.05, 0.3, 0.15)]     # the input is left alone
    # equal probabilities: the one with the smaller index comes first
    q = np.array([0.25, 0.25, 0.25, 0.25], dtype=np.float32)
    assert filter_top_p(q, 0.3).tolist() == [0.25, 0.25, 0, 0]


@pytest.mark.parametrize("seed", range(6))
def test_top_p_is_the_reference_s_loop(seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(2, 3000))
    logits = rng.normal(size=n) * rng.uniform(0.5, 6.0)
    probs = np.exp(logits - logits.max())
    probs = (probs / probs.sum()).astype(np.float32)
    if seed % 2:
        probs[rng.integers(0, n, size=n // 3)] = probs[0]                    # ties
    for top_p in (0.0, 0.1, 0.5, 0.9, 0.999, 1.0):
        assert np.array_equal(filter_top_p(probs, top_p), _top_p_by_the_book(probs, top_p)), top_p


def test_top_k():
    p = np.array([0.1, 0.4, 0.05, 0.3, 0.15], dtype=np.float32)
    assert filter_top_k(p, 2).tolist() == [0, p[1], 0, p[3], 0]
    assert filter_top_k(p, 5) is p and filter_top_k(p, 9) is p
    q = np.array([0.2, 0.3, 0.3, 0.2], dtype=np.float32)
    assert filter_top_k(q, 1).tolist() == [0, q[1], 0, 0] and filter_top_k(q, 3).tolist() == [q[0], q[1], q[2], 0]


def test_draw_walks_the_weights_in_index_order():
    p = np.array([0.0, 0.5, 0.0, 0.25, 0.25], dtype=np.float32)
    assert [draw(p, u) for u in (0.0, 0.49, 0.5, 0.74, 0.75, 0.999999)] == [1, 1, 3, 3, 4, 4]
    assert draw(p * 4.0, 0.6) == 3                                             # weights need not add up to one
    assert draw(np.array([0.3, 0.7, 0.0, 0.0], dtype=np.float32), 0.9999999999) == 1   # never a token of weight zero
    assert draw(np.zeros(4, dtype=np.float32), 0.3) == 0
    # frequencies follow the weights
    rng = np.random.default_rng(0)
    counts = np.bincount([draw(p, u) for u in rng.random(20000)], minlength=5) / 20000
    assert np.abs(counts - p).max() < 0.01
