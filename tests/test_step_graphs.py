"""Steps with prompt tokens replayed from captured pieces: the same logits as the same steps launched kernel by
kernel, through mixed schedules with so few pages that they are used again."""
import pytest
import torch

import harness
import tiny


def test_buckets_cover_their_token_counts():
    from prelude_b200.engine.step_graph import bucket_of
    last = 0
    for n in range(1, 9000):
        b = bucket_of(n)
        assert b >= n and b >= last and b - n < max(32, n // 4), (n, b)      # never more than a quarter of padding
        last = b
    assert bucket_of(1) == 32 and bucket_of(32) == 32 and bucket_of(33) == 64 and bucket_of(257) == 320
    assert bucket_of(1024) == 1024 and bucket_of(1025) == 1152 and bucket_of(4097) == 4352


def _runners(folder, dtype, page, graphs):
    from prelude_b200.engine.loading import load_model, make_runner
    model = load_model(folder, dtype, "cuda:0")
    runner = make_runner(model, page_size=page, num_pages=40 * 8 // page + 8, max_slots=8, max_request_tokens=512)
    if graphs:
        assert runner.enable_step_graphs(512)
    return runner


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["B", "D", "E"])
def test_captured_steps_give_the_logits_of_launched_steps(tmp_path, which, dtype):
    cfg, _, page = tiny.PARAMS[which]
    folder = tiny.make_folder(tmp_path, which, dtype)
    reqs = {f"r{i}": tiny.random_ids(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([70, 45, 133, 100, 64, 20])}
    outs = {}
    for graphs in (False, True):
        runner = _runners(folder, dtype, page, graphs)
        for rep in range(2):                   # the second pass replays what the first captured
            outs[(graphs, rep)] = harness.run_schedule(runner, harness.mixed(reqs, max_live=4, seed=3 + rep))
        runner.cache.check()
        assert runner.cache.used_pages() == 0
        if graphs:
            assert runner.graph_steps_run > 0.5 * runner.steps_run
            assert sum(g.replays for g in runner.step_graphs.graphs.values()) > 0.4 * runner.steps_run
    for rep in range(2):
        for key, row in outs[(False, rep)].items():
            other = outs[(True, rep)][key]
            if dtype == torch.float32:
                assert torch.equal(row, other), key            # the same kernels in the same order on every row
            else:
                # a padded step may take another product kernel (more rows): rounding differs, nothing else
                assert float((row - other).abs().max()) <= 3e-2 * float(row.abs().max()), key


@pytest.mark.gpu
def test_a_step_longer_than_the_limit_is_launched(tmp_path):
    cfg, _, page = tiny.PARAMS["E"]
    folder = tiny.make_folder(tmp_path, "E", torch.bfloat16)
    from prelude_b200.engine.loading import load_model, make_runner
    from prelude_b200.engine.runner import StepEntry
    model = load_model(folder, torch.bfloat16, "cuda:0")
    runner = make_runner(model, page_size=page, num_pages=100, max_slots=4, max_request_tokens=400)
    assert runner.enable_step_graphs(64)
    toks = tiny.random_ids(200, cfg["vocab_size"], 5)
    a = runner.step([StepEntry("a", toks[:100], [99])])       # 100 tokens: over the limit of 64
    assert runner.graph_steps_run == 0
    b = runner.step([StepEntry("a", toks[100:150], [49])])    # 50 tokens: captured at 64
    assert runner.graph_steps_run == 1 and sorted(runner.step_graphs.graphs) == [64]
    c = runner.step([StepEntry("a", toks[150:151], [0])])     # a decode step is not a prompt step
    assert runner.graph_steps_run == 1
    assert a.shape == b.shape == c.shape == (1, cfg["vocab_size"])
    # without the device-resident block tables there is nothing to capture against
    plain = make_runner(model, page_size=page, num_pages=100, max_slots=4)
    assert not plain.enable_step_graphs(64)


@pytest.mark.gpu
def test_engine_warms_up_and_generates_the_same_tokens(tmp_path):
    from prelude_b200 import Engine
    cfg = tiny.PARAMS["E"][0]
    folder = tiny.make_folder(tmp_path, "E", torch.float32)
    prompts = [tiny.random_ids(n, cfg["vocab_size"], 11 + n) for n in (3, 40, 97, 150)]
    outs = []
    for graphs in (False, True):
        engine = Engine(folder, dtype="f32", device="cuda:0", page_size=8, num_pages=120, max_running_requests=4,
                        cuda_graph=graphs)
        if graphs:
            assert engine.warmup_prompt_steps([40, 100]) == [64, 128]
            assert engine.warmup_prompt_steps([40, 100]) == []          # already there
        else:
            assert engine.warmup_prompt_steps([40, 100]) == []
        one_by_one = [engine.generate(p, temperature=0.0, max_new_tokens=5, ignore_eos=True).token_ids for p in prompts]
        together = [r.token_ids for r in engine.generate(prompts, temperature=0.0, max_new_tokens=5, ignore_eos=True)]
        assert one_by_one == together
        outs.append(together)
        if graphs:
            assert engine.runner.graph_steps_run >= 4
        engine.cache.check()
    assert outs[0] == outs[1]                  # 32-bit: the same kernels on every row, captured or launched


@pytest.mark.gpu
def test_a_recording_that_fails_leaves_no_capture_open(tmp_path, monkeypatch):
    cfg, _, page = tiny.PARAMS["E"]
    folder = tiny.make_folder(tmp_path, "E", torch.bfloat16)
    from prelude_b200.engine.loading import load_model, make_runner
    from prelude_b200.engine.runner import StepEntry
    from prelude_b200.parts import mlp
    model = load_model(folder, torch.bfloat16, "cuda:0")
    runner = make_runner(model, page_size=page, num_pages=100, max_slots=4, max_request_tokens=400)
    assert runner.enable_step_graphs(128)
    toks = tiny.random_ids(60, cfg["vocab_size"], 5)
    real = mlp.GatedMlp.forward
    calls = []

    def failing(self, x):
        calls.append(1)
        if len(calls) == 2:                                   # in the second layer, in the middle of a piece
            raise RuntimeError("made to fail")
        return real(self, x)
    monkeypatch.setattr(mlp.GatedMlp, "forward", failing)
    with pytest.raises(RuntimeError, match="made to fail"):
        runner.step([StepEntry("a", toks[:40], [39])])
    assert not torch.cuda.is_current_stream_capturing()
    monkeypatch.setattr(mlp.GatedMlp, "forward", real)
    runner.finish("a")
    want = runner.step([StepEntry("b", toks[:40], [39])])     # the bucket is launched kernel by kernel from now on
    assert runner.graph_steps_run == 0 and runner.step_graphs.graphs[64].failed
    runner.finish("b")
    other = make_runner(model, page_size=page, num_pages=100, max_slots=4)
    got = other.step([StepEntry("b", toks[:40], [39])])
    assert torch.equal(want, got)


@pytest.mark.gpu
def test_graphs_of_a_dropped_engine_are_not_collected_inside_a_capture(tmp_path):
    # An engine that is no longer used leaves its captured graphs in reference cycles.  The cycle collector must
    # not free them while another engine records: destroying a graph during a capture invalidates the capture.
    # With the collector's threshold at its lowest it would run at almost every allocation of the recording.
    import gc
    from prelude_b200 import Engine
    cfg = tiny.PARAMS["E"][0]
    folder = tiny.make_folder(tmp_path, "E", torch.bfloat16)
    prompts = [tiny.random_ids(n, cfg["vocab_size"], 5 + n) for n in (40, 70)]

    def run():
        engine = Engine(folder, dtype="bf16", device="cuda:0", page_size=16, num_pages=64, max_running_requests=4)
        out = [r.token_ids for r in engine.generate(prompts, temperature=0.0, max_new_tokens=6, ignore_eos=True)]
        assert engine.runner.graph_steps_run >= 1
        holder = {"engine": engine}
        holder["self"] = holder                  # a cycle: only the collector frees this engine and its graphs
        return out

    old = gc.get_threshold()
    gc.disable()                                 # the garbage of the first run stays until a collection is asked for
    try:
        first = run()
        gc.enable()
        gc.set_threshold(1, 1, 1)
        second = run()
    finally:
        gc.set_threshold(*old)
        gc.enable()
    assert first == second
