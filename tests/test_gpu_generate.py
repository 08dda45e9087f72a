"""Generation through the Python entry point and the command line: greedy against
the plain implementation, seeded sampling, page pressure, long decoding."""
import json
import os
import subprocess
import sys

import pytest
import torch

import tiny
from plain.qwen3_plain import forward_logits, greedy_generate

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {w: tiny.make_folder(root, w, torch.float32) for w in "ABC"}


def _engine(folder, dtype="f32", **kw):
    from prelude_b200 import Engine
    args = dict(dtype=dtype, device="cuda:0", page_size=4, num_pages=64, max_running_requests=8)
    args.update(kw)
    return Engine(folder, **args)


def _prompts(which, lens):
    v = tiny.PARAMS[which][0]["vocab_size"]
    return [tiny.random_ids(n, v, 50 + n) for n in lens]


@pytest.mark.parametrize("which,lens,new", [("A", [1, 5, 17], 8), ("B", [2, 9, 31, 64], 12), ("C", [40, 3], 10)])
def test_greedy_tokens_equal_the_plain_implementation_in_32_bit(folders, which, lens, new):
    cfg = tiny.PARAMS[which][0]
    w = tiny.read_weights(folders[which])
    prompts = _prompts(which, lens)
    want = [greedy_generate(cfg, w, p, new) for p in prompts]
    eng = _engine(folders[which], page_size=tiny.PARAMS[which][2])
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    assert all(r.finish_reason == "length" and r.completion_tokens == new for r in got)
    assert [r.prompt_tokens for r in got] == lens
    # one at a time, and cut into small portions beside decoding requests: the same tokens
    assert [eng.generate(p, temperature=0.0, max_new_tokens=new, ignore_eos=True).token_ids for p in prompts] == want
    eng2 = _engine(folders[which], page_size=tiny.PARAMS[which][2], max_num_batched_tokens=7, long_prefill_token_threshold=3)
    assert [r.token_ids for r in eng2.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want
    assert eng.cache.used_pages() == 0 and eng2.cache.used_pages() == 0


@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_in_bfloat16_picks_tokens_the_plain_implementation_rates_near_its_best(folders, which, tmp_path):
    cfg = tiny.PARAMS[which][0]
    folder = tiny.make_folder(tmp_path, which, torch.bfloat16)
    w = tiny.read_weights(folder)
    prompts = _prompts(which, [5, 17, 30])
    eng = _engine(folder, dtype="bf16", page_size=tiny.PARAMS[which][2])
    for p, r in zip(prompts, eng.generate(prompts, temperature=0.0, max_new_tokens=10, ignore_eos=True)):
        logits = forward_logits(cfg, w, p + r.token_ids)          # teacher-forced on what the engine chose
        for i, tok in enumerate(r.token_ids):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 3e-2 * float(row.abs().max())


def test_long_decoding_stays_on_the_plain_implementation(folders):
    cfg = tiny.PARAMS["C"][0]
    w = tiny.read_weights(folders["C"])
    prompt = _prompts("C", [7])[0]
    want = greedy_generate(cfg, w, prompt, 150)
    eng = _engine(folders["C"], page_size=16, num_pages=12)
    assert eng.generate(prompt, temperature=0.0, max_new_tokens=150, ignore_eos=True).token_ids == want


def test_eos_and_stop_tokens_end_a_request(folders):
    cfg = tiny.PARAMS["B"][0]                                      # eos_token_id [7, 9] in its config.json
    w = tiny.read_weights(folders["B"])
    prompt = _prompts("B", [9])[0]
    free = greedy_generate(cfg, w, prompt, 12)
    eng = _engine(folders["B"], page_size=8)
    r = eng.generate(prompt, temperature=0.0, max_new_tokens=12, stop_token_ids=[free[4]])
    cut = min(i for i, t in enumerate(free) if t == free[4] or t in (7, 9))
    assert r.token_ids == free[:cut + 1] and r.finish_reason in ("stop", "eos")
    assert eng.eos_token_ids == (7, 9)


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(folders):
    eng = _engine(folders["B"], page_size=8)
    prompts = _prompts("B", [2, 9, 31, 64])
    a = eng.generate(prompts, temperature=0.8, seed=11, max_new_tokens=12, ignore_eos=True)
    b = eng.generate(prompts, temperature=0.8, seed=11, max_new_tokens=12, ignore_eos=True)
    c = eng.generate(prompts, temperature=0.8, seed=12, max_new_tokens=12, ignore_eos=True)
    assert [r.token_ids for r in a] == [r.token_ids for r in b] != [r.token_ids for r in c]
    alone = eng.generate(prompts[2], temperature=0.8, seed=11, max_new_tokens=12, ignore_eos=True)
    assert alone.token_ids == a[2].token_ids
    greedy = eng.generate(prompts, temperature=0.0, max_new_tokens=12, ignore_eos=True)
    assert [r.token_ids for r in greedy] != [r.token_ids for r in a]
    # top-k = 1 is greedy whatever the temperature; top-p and top-k runs are seeded too
    k1 = eng.generate(prompts, temperature=0.9, top_k=1, max_new_tokens=12, ignore_eos=True)
    assert [r.token_ids for r in k1] == [r.token_ids for r in greedy]
    p1 = eng.generate(prompts, temperature=0.9, top_p=0.5, top_k=20, seed=3, max_new_tokens=6, ignore_eos=True)
    p2 = eng.generate(prompts, temperature=0.9, top_p=0.5, top_k=20, seed=3, max_new_tokens=6, ignore_eos=True)
    assert [r.token_ids for r in p1] == [r.token_ids for r in p2]


def test_queued_runs_of_decode_steps_give_the_tokens_of_single_steps(folders):
    """With decode_burst > 1 the engine queues several decode steps and reads their tokens at the end;
    requests of different lengths, stops in the middle of a run and seeded sampling come out the same
    as with one step at a time."""
    prompts = _prompts("B", [2, 9, 31, 64])
    single, burst = _engine(folders["B"], page_size=8, decode_burst=1), _engine(folders["B"], page_size=8, decode_burst=5)
    for kw in (dict(temperature=0.0, max_new_tokens=13, ignore_eos=True),
               dict(temperature=0.8, seed=5, max_new_tokens=11, ignore_eos=True),
               dict(temperature=0.0, max_new_tokens=12)):                       # eos ids 7 and 9 may cut requests short
        a, b = single.generate(prompts, **kw), burst.generate(prompts, **kw)
        assert [r.token_ids for r in a] == [r.token_ids for r in b]
        assert [r.finish_reason for r in a] == [r.finish_reason for r in b]
    assert burst.stats().graph_steps > 0 and burst.cache.used_pages() == 0
    # a stop token in the middle of a run: the tokens after it are dropped
    free = single.generate(prompts[1], temperature=0.0, max_new_tokens=12, ignore_eos=True).token_ids
    a = single.generate(prompts[1], temperature=0.0, max_new_tokens=12, ignore_eos=True, stop_token_ids=[free[3]])
    b = burst.generate(prompts[1], temperature=0.0, max_new_tokens=12, ignore_eos=True, stop_token_ids=[free[3]])
    assert a.token_ids == b.token_ids and b.finish_reason == "stop" and len(b.token_ids) <= 4
    # different lengths to go: the run is as long as the shortest, the rest goes on afterwards
    params = [dict(max_new_tokens=n) for n in (3, 9, 14, 6)]
    from prelude_b200 import SamplingParams
    sp = [SamplingParams(temperature=0.0, ignore_eos=True, **p) for p in params]
    a, b = single.generate(prompts, sp), burst.generate(prompts, sp)
    assert [r.token_ids for r in a] == [r.token_ids for r in b] and [len(r.token_ids) for r in b] == [3, 9, 14, 6]


def test_when_pages_run_out_requests_are_preempted_and_still_get_the_same_tokens(folders):
    cfg = tiny.PARAMS["A"][0]
    w = tiny.read_weights(folders["A"])
    prompts = _prompts("A", [9, 10, 11, 12])
    want = [greedy_generate(cfg, w, p, 20) for p in prompts]
    # 4 requests of up to 32 tokens need 32 pages of 4; 14 pages force preemption
    eng = _engine(folders["A"], page_size=4, num_pages=14, decode_reservation_cap=1)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=20, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    assert sum(r.preemptions for r in got) >= 1 and eng.stats().preemptions >= 1
    assert eng.cache.used_pages() == 0
    eng.cache.check()
    # a request that cannot fit even alone ends with cache_full instead of hanging
    r = _engine(folders["A"], page_size=4, num_pages=4).generate(prompts[0], temperature=0.0, max_new_tokens=40, ignore_eos=True)
    assert r.finish_reason == "cache_full" and r.token_ids == want[0][:len(r.token_ids)] and len(r.token_ids) == 8


def test_bad_requests_are_refused(folders):
    eng = _engine(folders["A"])
    with pytest.raises(ValueError, match="token ids"):
        eng.generate([1, 2, 256])
    with pytest.raises(ValueError):
        eng.generate([list(range(128))])
    with pytest.raises(ValueError):
        _engine(folders["A"], dtype="fp8")


def test_command_line(folders):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "prelude"), "--model", folders["A"], "--dtype", "f32",
                          "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6", "--max-new-tokens", "5",
                          "--temperature", "0", "--num-pages", "16", "--page-size", "4", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(line) for line in out.stdout.strip().splitlines()]
    cfg, w = tiny.PARAMS["A"][0], tiny.read_weights(folders["A"])
    assert [r["token_ids"] for r in lines] == [greedy_generate(cfg, w, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    assert lines[0]["finish_reason"] == "length" and lines[0]["usage"] == {"prompt_tokens": 3, "completion_tokens": 5}
    # whole prompts only, one decode step at a time, device from the environment: the same tokens
    env = dict(os.environ, PRELUDE_DEVICE="cuda:0")
    out2 = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "prelude"), "--model-path", folders["A"], "--dtype", "f32",
                           "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6", "--max-tokens", "5", "--temperature", "0",
                           "--num-pages", "16", "--page-size", "4", "--ignore-eos", "--no-chunked-prefill",
                           "--max-num-batched-tokens", "2", "--decode-burst", "1"],
                          capture_output=True, text=True, timeout=600, env=env)
    assert out2.returncode == 0, out2.stderr
    assert [json.loads(line)["token_ids"] for line in out2.stdout.strip().splitlines()] == [r["token_ids"] for r in lines]
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "prelude"), "--model", folders["A"], "--device", "cpu",
                          "--prompt-ids", "1"], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "no cpu path" in bad.stderr


def test_random_weights_from_a_seed_need_the_configuration_alone(folders, tmp_path):
    # a folder with config.json and nothing else: --random-weights draws the tensors the model asks for from --seed
    # on the device; the same seed gives the same tokens, through the command line and through the entry point
    import shutil
    from prelude_b200 import Engine
    from prelude_b200.weights.random_init import random_tensors
    bare = tmp_path / "bare"
    bare.mkdir()
    shutil.copy(os.path.join(folders["B"], "config.json"), bare / "config.json")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "prelude"), "--model", str(bare), "--dtype", "f32", "--random-weights",
           "--seed", "7", "--prompt-ids", "5,17,3,9", "--max-new-tokens", "6", "--temperature", "0", "--num-pages", "16", "--ignore-eos"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    tokens = json.loads(out.stdout.strip().splitlines()[0])["token_ids"]
    eng = Engine(str(bare), dtype="f32", num_pages=16, random_weights_seed=7)
    assert eng.generate([5, 17, 3, 9], temperature=0.0, max_new_tokens=6, ignore_eos=True).token_ids == tokens
    # and they are the plain implementation's tokens for those tensors
    cfg = json.load(open(bare / "config.json"))
    w = {k: v.cpu() for k, v in random_tensors(cfg, seed=7, std=0.02, norm_jitter=0.05, dtype=torch.float32, device="cuda:0").items()}
    assert tokens == greedy_generate(cfg, w, [5, 17, 3, 9], 6)
    missing = subprocess.run(cmd[:6] + cmd[7:], capture_output=True, text=True, timeout=600)       # without --random-weights
    assert missing.returncode != 0 and "safetensors" in missing.stderr


def test_a_generation_that_fails_gives_its_pages_back(folders, monkeypatch):
    # a step that raises in the middle of a generation: the call raises, nothing stays held, the engine goes on
    cfg, w = tiny.PARAMS["A"][0], tiny.read_weights(folders["A"])
    eng = _engine(folders["A"], cuda_graph=False)
    prompts = _prompts("A", [9, 17, 5])
    step, calls = eng.runner.step, []

    def failing(entries, **kw):
        calls.append(len(entries))
        if len(calls) == 3:
            raise RuntimeError("made to fail")
        return step(entries, **kw)

    monkeypatch.setattr(eng.runner, "step", failing)
    with pytest.raises(RuntimeError, match="made to fail"):
        eng.generate(prompts, temperature=0.0, max_new_tokens=6, ignore_eos=True)
    assert len(calls) == 3
    eng.cache.check()
    assert eng.cache.used_pages() == 0 and not eng.cache.requests
    monkeypatch.setattr(eng.runner, "step", step)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=6, ignore_eos=True)
    assert [r.token_ids for r in got] == [greedy_generate(cfg, w, p, 6) for p in prompts]
