"""The engine against the plain implementation, on the GPU, in 32-bit and in
bfloat16: whole requests, a decoded tail, changing portions, and mixed batches
with so few pages that they are used again."""
import pytest
import torch

import harness
import tiny
from plain.qwen3_plain import forward_logits

pytestmark = pytest.mark.gpu

# bfloat16 has 8 bits of mantissa; through a few layers the logits of these
# models stay within 3% of their largest magnitude.  32-bit differs from the
# plain implementation by summation order only.
TOL = {torch.float32: (1e-4, 0.0), torch.bfloat16: (0.0, 3e-2)}

REQUESTS = {
    "A": {"a1": 1, "a5": 5, "a17": 17, "a70": 70},
    "B": {"b2": 2, "b9": 9, "b31": 31, "b64": 64, "b150": 150},
    "C": {"c40": 40, "c33": 33, "c129": 129},
    "D": {"d3": 3, "d70": 70, "d200": 200},
    "E": {"e2": 2, "e45": 45, "e130": 130, "e300": 300},
}


def _requests(which):
    cfg = tiny.PARAMS[which][0]
    return {rid: tiny.random_ids(n, cfg["vocab_size"], sum(map(ord, rid))) for rid, n in REQUESTS[which].items()}


def _reference(which, folder, reqs):
    cfg = tiny.PARAMS[which][0]
    w = tiny.read_weights(folder)
    return {rid: forward_logits(cfg, w, toks) for rid, toks in reqs.items()}


def _compare(got, ref, dtype):
    atol, rel = TOL[dtype]
    worst = 0.0
    for (rid, pos), row in got.items():
        want = ref[rid][pos]
        bound = atol + rel * float(want.abs().max())
        diff = float((row - want).abs().max())
        worst = max(worst, diff / bound)
        assert diff <= bound, f"request {rid} position {pos}: max diff {diff:.3e} > {bound:.3e}"
    return worst


def _runner(folder, dtype, page_size, num_pages):
    from prelude_b200.engine.loading import load_model, make_runner
    model = load_model(folder, dtype, "cuda:0")
    return make_runner(model, page_size=page_size, num_pages=num_pages, max_slots=8)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for which in "ABCDE":
        for dtype in (torch.float32, torch.bfloat16):
            out[(which, dtype)] = tiny.make_folder(root, which, dtype)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_match_plain(folders, which, dtype, cut):
    folder = folders[(which, dtype)]
    reqs = _requests(which)
    ref = _reference(which, folder, reqs)
    page = tiny.PARAMS[which][2]
    schedule = {"whole": harness.whole, "tail_decode": harness.tail_decode, "portions": harness.portions,
                "mixed": harness.mixed}[cut](reqs)
    need = harness.peak_tokens(schedule, page)
    total = sum(-(-len(t) // page) for t in reqs.values())
    num_pages = need // page                      # exactly what the busiest moment needs
    if cut == "mixed":
        assert num_pages < total, "the pool must be smaller than the sum of all requests, so pages are used again"
    runner = _runner(folder, dtype, page, num_pages)
    got = harness.run_schedule(runner, schedule)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, ref, dtype)
    runner.cache.check()
    assert runner.cache.used_pages() == 0 and not runner.cache.requests


@pytest.mark.parametrize("which", ["A", "B"])
def test_f32_cuts_agree_bitwise(folders, which):
    """In 32-bit every kernel sums in an order that depends on the row alone, so
    all ways of cutting give the same bits."""
    folder = folders[(which, torch.float32)]
    reqs = _requests(which)
    page = tiny.PARAMS[which][2]
    results = []
    for cut in (harness.whole, harness.tail_decode, harness.portions, harness.mixed):
        schedule = cut(reqs)
        runner = _runner(folder, torch.float32, page, harness.peak_tokens(schedule, page) // page)
        results.append(harness.run_schedule(runner, schedule))
    for other in results[1:]:
        for key, row in results[0].items():
            assert torch.equal(row, other[key]), f"{key}: cuts disagree by {(row - other[key]).abs().max():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "C", "E"])
def test_the_first_tokens_of_a_sequence(folders, which, dtype):
    """A request fed token by token from an empty cache: the step at position 0 attends to one key, its own; the
    page table has one page, then a second when the first is full; and a second request starts in between, so
    that the first tokens of one sequence lie beside later tokens of another in the same step."""
    folder = folders[(which, dtype)]
    cfg, _, page = tiny.PARAMS[which]
    n = 2 * page + 3                                         # past the first page's edge and the second's
    reqs = {"p": tiny.random_ids(n, cfg["vocab_size"], 5), "q": tiny.random_ids(page + 2, cfg["vocab_size"], 6)}
    ref = _reference(which, folder, reqs)
    late = page - 1                                          # q's first token arrives beside p's last token of its first page
    schedule = []
    for i in range(n):
        entries = [("p", [reqs["p"][i]], [0])]
        j = i - late
        if 0 <= j < len(reqs["q"]):
            entries.append(("q", [reqs["q"][j]], [0]))
        schedule.append((entries, ["q"] if j == len(reqs["q"]) - 1 else []))
    schedule[-1] = (schedule[-1][0], schedule[-1][1] + ["p"])
    runner = _runner(folder, dtype, page, harness.peak_tokens(schedule, page) // page)
    got = harness.run_schedule(runner, schedule)
    assert len(got) == n + len(reqs["q"]) and ("p", 0) in got and ("q", 0) in got
    _compare(got, ref, dtype)
    runner.cache.check()
    assert runner.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["D", "E"])
def test_long_portions_behind_a_cached_prefix(folders, which, dtype):
    """Portions of 64 to 130 tokens that continue a cached prefix, alone and beside single decoded tokens of other
    requests: long enough for the tcgen05 prompt-attention kernel (where it takes the shape) to start in the
    middle of a request, with captured prompt steps on as in the entry point."""
    folder = folders[(which, dtype)]
    cfg, _, page = tiny.PARAMS[which]
    reqs = {"p": tiny.random_ids(330, cfg["vocab_size"], 31), "q": tiny.random_ids(200, cfg["vocab_size"], 32),
            "r": tiny.random_ids(90, cfg["vocab_size"], 33)}
    ref = _reference(which, folder, reqs)
    alone = harness.portions(reqs, sizes=(30, 70, 2, 130, 64, 3, 1))
    # mixed by hand: p's long portions beside q's and r's single tokens
    beside, fed = [], {"p": 0, "q": 0, "r": 0}
    beside.append(([("q", reqs["q"][:150], list(range(150))), ("r", reqs["r"][:60], list(range(60)))], []))
    fed["q"], fed["r"] = 150, 60
    for n in (33, 64, 100, 128, 5):
        entries = [("p", reqs["p"][fed["p"]:fed["p"] + n], list(range(n)))]
        fed["p"] += n
        for rid in ("q", "r"):
            if fed[rid] < len(reqs[rid]):
                entries.append((rid, reqs[rid][fed[rid]:fed[rid] + 1], [0]))
                fed[rid] += 1
        beside.append((entries, []))
    beside.append(([(rid, reqs[rid][fed[rid]:], list(range(len(reqs[rid]) - fed[rid]))) for rid in reqs
                    if fed[rid] < len(reqs[rid])], list(reqs)))
    for schedule in (alone, beside):
        from prelude_b200.engine.loading import load_model, make_runner
        model = load_model(folder, dtype, "cuda:0")
        runner = make_runner(model, page_size=page, num_pages=harness.peak_tokens(schedule, page) // page, max_slots=8,
                             max_request_tokens=512)
        runner.enable_step_graphs()
        got = harness.run_schedule(runner, schedule)
        assert len(got) == sum(len(t) for t in reqs.values())
        _compare(got, ref, dtype)
        runner.cache.check()
        assert runner.cache.used_pages() == 0
