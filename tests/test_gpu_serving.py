"""Requests that arrive and leave while the engine runs: ``submit``, ``step_once``, ``abort``,
``run_until_idle``.  Every request's tokens are those it gets alone (32-bit: bit-identical logits whatever the
batch), whenever it joins and whoever leaves beside it, and what an aborted request held comes back."""
import pytest
import torch

import tiny
from plain.qwen3_plain import greedy_generate

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return tiny.make_folder(tmp_path_factory.mktemp("serving"), "B", torch.float32)


def _engine(folder, **kw):
    from prelude_b200 import Engine
    args = dict(dtype="f32", device="cuda:0", page_size=8, num_pages=96, max_running_requests=8)
    args.update(kw)
    return Engine(folder, **args)


def _prompts(lens):
    v = tiny.PARAMS["B"][0]["vocab_size"]
    return [tiny.random_ids(n, v, 70 + n) for n in lens]


def _plain(folder, prompts, new):
    cfg, w = tiny.PARAMS["B"][0], tiny.read_weights(folder)
    return [greedy_generate(cfg, w, p, new) for p in prompts]


@pytest.mark.parametrize("burst", [1, 6])
def test_a_request_that_arrives_while_others_run_gets_the_tokens_it_gets_alone(folder, burst):
    prompts = _prompts([5, 40, 9, 23, 64])
    new = 14
    want = _plain(folder, prompts, new)
    eng = _engine(folder, decode_burst=burst, max_num_batched_tokens=16)     # prompts are cut into portions
    ids, results, steps = [], {}, 0
    while len(results) < len(prompts):
        if len(ids) < len(prompts) and steps >= 3 * len(ids):                 # request k arrives after step 3 k
            ids.append(eng.submit(prompts[len(ids)], temperature=0.0, max_new_tokens=new, ignore_eos=True))
        for r in eng.step_once():
            results[r.request_id] = r
        steps += 1
        assert steps < 400
    assert [results[i].token_ids for i in ids] == want
    assert all(results[i].finish_reason == "length" for i in ids)
    assert not eng.has_work() and eng.cache.used_pages() == 0 and not eng.cache.requests
    eng.cache.check()
    # the engine is the same one afterwards: a plain generate call on it
    assert [r.token_ids for r in eng.generate(prompts[:2], temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want[:2]


def test_abort_in_the_middle_of_a_prompt_and_in_the_middle_of_decoding(folder):
    prompts = _prompts([60, 12, 33, 50])
    new = 12
    want = _plain(folder, prompts, new)
    eng = _engine(folder, max_num_batched_tokens=8, decode_burst=1)           # 60 tokens take eight steps
    ids = [eng.submit(p, temperature=0.0, max_new_tokens=new, ignore_eos=True) for p in prompts]
    results = {}

    def step():
        for r in eng.step_once():
            results[r.request_id] = r

    step()
    step()
    seq0 = next(s for s in eng.sched.running if s.request_id == ids[0])
    assert 0 < seq0.computed < len(prompts[0])                                # in the middle of its prompt
    held = eng.cache.used_pages()
    eng.abort(ids[0])
    step()
    assert results[ids[0]].finish_reason == "abort" and results[ids[0]].token_ids == []
    assert not eng.cache.has_request(ids[0]) and eng.cache.used_pages() < held + 4
    eng.cache.check()
    # run on until request 1 is decoding, then abort it
    while not any(s.request_id == ids[1] and len(s.output) >= 3 for s in eng.sched.running):
        step()
    eng.abort(ids[1])
    eng.abort(12345)                                                          # unknown ids are ignored
    step()
    r1 = results[ids[1]]
    assert r1.finish_reason == "abort" and 3 <= len(r1.token_ids) < new and r1.token_ids == want[1][:len(r1.token_ids)]
    eng.cache.check()
    for r in eng.run_until_idle():
        results[r.request_id] = r
    # the others never noticed
    assert results[ids[2]].token_ids == want[2] and results[ids[3]].token_ids == want[3]
    assert eng.cache.used_pages() == 0 and not eng.cache.requests and not eng.has_work()
    eng.cache.check()
    # an abort of a request that is still waiting (never admitted)
    a = eng.submit(prompts[0], temperature=0.0, max_new_tokens=4, ignore_eos=True)
    eng.abort(a)
    out = eng.run_until_idle()
    assert [(r.request_id, r.finish_reason) for r in out] == [(a, "abort")] and eng.cache.used_pages() == 0


def test_a_run_of_queued_decode_steps_is_cut_short_when_a_request_arrives(folder):
    prompts = _prompts([9, 31, 17])
    new = 30
    want = _plain(folder, prompts, new)
    eng = _engine(folder, decode_burst=8)
    ids = [eng.submit(p, temperature=0.0, max_new_tokens=new, ignore_eos=True) for p in prompts[:2]]
    results, runs = {}, []
    from prelude_b200.engine.graph import DecodeGraph
    replay_burst = DecodeGraph.replay_burst
    replays = {"n": 0}
    replay = DecodeGraph.replay

    def counting_replay(self):
        replays["n"] += 1 if self.self_feeding else 0
        if self.self_feeding and replays["n"] == 2 and len(ids) == 2:
            # while a run of eight is being queued (at its second replay), another request is handed in
            ids.append(eng.submit(prompts[2], temperature=0.0, max_new_tokens=new, ignore_eos=True))
        return replay(self)

    def recording_burst(self, steps, stop=None, ahead=3):
        out = replay_burst(self, steps, stop, ahead)
        runs.append((steps, len(out)))
        return out

    DecodeGraph.replay, DecodeGraph.replay_burst = counting_replay, recording_burst
    try:
        while eng.has_work():
            for r in eng.step_once():
                results[r.request_id] = r
    finally:
        DecodeGraph.replay, DecodeGraph.replay_burst = replay, replay_burst
    assert len(ids) == 3 and [results[i].token_ids for i in ids] == want
    assert any(ran < asked for asked, ran in runs), f"no run was cut short: {runs}"
    assert any(ran == asked for asked, ran in runs)
    assert eng.cache.used_pages() == 0 and not eng.cache.requests
    eng.cache.check()


def test_results_of_requests_that_are_not_generates_own_are_kept(folder):
    prompts = _prompts([7, 15])
    want = _plain(folder, prompts, 6)
    eng = _engine(folder)
    other = eng.submit(prompts[1], temperature=0.0, max_new_tokens=6, ignore_eos=True)
    mine = eng.generate(prompts[0], temperature=0.0, max_new_tokens=6, ignore_eos=True)
    assert mine.token_ids == want[0]
    for r in eng.run_until_idle():
        eng._done[r.request_id] = r
    assert eng.result(other).token_ids == want[1] and eng.result(other) is None
    with pytest.raises(TypeError):
        eng.submit(prompts[0], temperatur=0.0)


@pytest.mark.parametrize("burst,pages,seed", [(6, 72, 1), (1, 18, 5), (8, 24, 9)])
def test_random_arrivals_aborts_sampling_and_page_pressure(folder, burst, pages, seed):
    """Some hundred requests that come at random steps, a few of them aborted at random moments, a fifth of them
    sampled (with and without filters) beside the greedy ones, a pool small enough in two of the three runs that
    requests are preempted: every greedy request that finishes has the tokens it gets alone from the plain
    implementation (an aborted one a prefix of them), nothing is held at the end.  Where a token differs, the plain
    implementation's float64 logits of the two candidates must be a tie (within 5e-5): among thousands of tokens of a
    flat random model that happens."""
    import random
    from plain.qwen3_plain import forward_logits
    cfg, w = tiny.PARAMS["B"][0], tiny.read_weights(folder)
    v = cfg["vocab_size"]
    rng = random.Random(seed)
    eng = _engine(folder, page_size=8, num_pages=pages, max_running_requests=6, max_num_batched_tokens=24, decode_burst=burst)
    cache, live = {}, {}
    submitted = checked = ties = aborted = steps = 0

    def plain(p, n):
        key = (tuple(p), n)
        if key not in cache:
            cache[key] = greedy_generate(cfg, w, p, n)
        return cache[key]

    while submitted < 160 or eng.has_work():
        if submitted < 160 and rng.random() < 0.35 and len(live) < 14:
            p = tiny.random_ids(rng.choice([1, 2, 3, 7, 8, 9, 15, 16, 17, 30, 45, 64, 90]), v, rng.randrange(1 << 20))
            new, greedy = rng.choice([1, 2, 5, 9, 16, 25]), rng.random() < 0.8
            extra = {} if greedy else {"top_k": rng.choice([None, 5]), "top_p": rng.choice([1.0, 0.9])}
            rid = eng.submit(p, temperature=0.0 if greedy else 0.9, seed=rng.randrange(1000), max_new_tokens=new, ignore_eos=True, **extra)
            live[rid] = (p, new, greedy)
            submitted += 1
        if live and rng.random() < 0.05:
            eng.abort(rng.choice(list(live)))
        for r in eng.step_once():
            p, new, greedy = live.pop(r.request_id)
            if r.finish_reason == "cache_full":
                continue
            if r.finish_reason == "abort":
                aborted += 1
            else:
                assert r.finish_reason == "length" and len(r.token_ids) == new
            if greedy:
                want = plain(p, new)[:len(r.token_ids)]
                if r.token_ids != want:
                    k = next(i for i in range(len(want)) if r.token_ids[i] != want[i])
                    lg = forward_logits(cfg, w, p + want[:k], dtype=torch.float64)[-1]
                    assert abs(float(lg[want[k]] - lg[r.token_ids[k]])) < 5e-5, (r.request_id, k, r.token_ids, want)
                    ties += 1
                checked += 1
        steps += 1
        assert steps < 20000
        if steps % 100 == 0:
            eng.cache.check()
    eng.cache.check()
    assert eng.cache.used_pages() == 0 and not eng.cache.requests and not live
    assert checked > 80 and ties <= 2 and aborted > 0
    if pages < 30:
        assert eng.stats().preemptions > 0
