"""The command line on the host, with a stand-in for the engine: the reference's option names
(crates/prelude-server/src/main.rs:15-183) and environment variables reach the engine under their meanings."""
import json

import pytest

import tiny


class _Result:
    def __init__(self, rid, toks):
        self.request_id, self.token_ids, self.finish_reason = rid, toks, "length"
        self.prompt_tokens, self.completion_tokens, self.ttft_ms, self.total_ms = len(toks), 1, 1.0, 2.0


@pytest.fixture
def fake_engine(monkeypatch):
    from prelude_b200.engine import engine as engine_module
    seen = {}

    class Engine:
        def __init__(self, model, **kw):
            seen["model"], seen["kw"] = model, kw

        def generate(self, prompts, params):
            seen["prompts"], seen["params"] = prompts, params
            return [_Result(i, p) for i, p in enumerate(prompts)]

    monkeypatch.setattr(engine_module, "Engine", Engine)
    return seen


def test_defaults_are_the_reference_s(fake_engine, capsys, monkeypatch):
    from prelude_b200.engine import cli
    for name in ("PRELUDE_DEVICE", "PRELUDE_PAGED_BLOCK_SIZE", "PRELUDE_PAGED_ATTN_BLOCKS", "PRELUDE_CUDA_GRAPH_MAX_BS",
                 "PRELUDE_DEFAULT_TEMPERATURE", "PRELUDE_DEFAULT_TOP_P", "PRELUDE_DEFAULT_MAX_TOKENS"):
        monkeypatch.delenv(name, raising=False)
    assert cli.main(["--model", "m", "--prompt-ids", "1,2 3", "--prompt-ids", "7"]) == 0
    kw, p = fake_engine["kw"], fake_engine["params"]
    assert fake_engine["model"] == "m" and fake_engine["prompts"] == [[1, 2, 3], [7]]
    assert kw["dtype"] == "bf16" and kw["device"] == "cuda:0" and kw["num_pages"] is None and kw["max_model_len"] is None
    assert (kw["max_running_requests"], kw["max_num_batched_tokens"], kw["long_prefill_token_threshold"]) == (256, 8192, 0)
    assert (kw["max_total_tokens"], kw["decode_reservation_cap"], kw["decode_priority_max_remaining_tokens"]) == (0, 0, 4)
    assert kw["gpu_memory_utilization"] == 0.9 and kw["cuda_graph"] is True and kw["cuda_graph_max_bs"] == 64
    assert (p.temperature, p.top_p, p.top_k, p.seed, p.max_new_tokens, p.stop_token_ids, p.ignore_eos) == (0.7, 1.0, None, 42, 4096, (), False)
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert [r["token_ids"] for r in lines] == [[1, 2, 3], [7]] and lines[0]["usage"] == {"prompt_tokens": 3, "completion_tokens": 1}


def test_options_and_environment(fake_engine, tmp_path, monkeypatch):
    from prelude_b200.engine import cli
    monkeypatch.setenv("PRELUDE_DEVICE", "cuda:0")
    monkeypatch.setenv("PRELUDE_PAGED_BLOCK_SIZE", "128")
    monkeypatch.setenv("PRELUDE_PAGED_ATTN_BLOCKS", "77")
    monkeypatch.setenv("PRELUDE_CUDA_GRAPH_MAX_BS", "32")
    monkeypatch.setenv("PRELUDE_DEFAULT_TEMPERATURE", "0.25")
    monkeypatch.setenv("PRELUDE_DEFAULT_TOP_P", "0.5")
    monkeypatch.setenv("PRELUDE_DEFAULT_MAX_TOKENS", "9")
    prompts = tmp_path / "p.txt"
    prompts.write_text("4 5 6\n\n8,9\n")
    assert cli.main(["--model-path", "m", "--dtype", "f32", "--prompt-file", str(prompts), "--max-running-requests", "3",
                     "--max-num-batched-tokens", "64", "--long-prefill-token-threshold", "16", "--max-total-tokens", "500",
                     "--decode-reservation-cap", "40", "--decode-priority-max-remaining-tokens", "2", "--no-cuda-graph",
                     "--gpu-memory-utilization", "0.5", "--top-k", "5", "--seed", "3", "--stop-token-ids", "1,2",
                     "--ignore-eos", "--max-model-len", "100", "--decode-burst", "1"]) == 0
    kw, p = fake_engine["kw"], fake_engine["params"]
    assert fake_engine["prompts"] == [[4, 5, 6], [8, 9]]
    assert kw["dtype"] == "f32" and kw["page_size"] == 128 and kw["num_pages"] == 77 and kw["cuda_graph_max_bs"] == 32
    assert (kw["max_running_requests"], kw["max_num_batched_tokens"], kw["long_prefill_token_threshold"]) == (3, 64, 16)
    assert (kw["max_total_tokens"], kw["decode_reservation_cap"], kw["decode_priority_max_remaining_tokens"]) == (500, 40, 2)
    assert kw["cuda_graph"] is False and kw["gpu_memory_utilization"] == 0.5 and kw["max_model_len"] == 100 and kw["decode_burst"] == 1
    assert (p.temperature, p.top_p, p.top_k, p.seed, p.max_new_tokens, p.stop_token_ids, p.ignore_eos) == (0.25, 0.5, 5, 3, 9, (1, 2), True)


def test_whole_prompts_only_raises_the_budget_to_the_longest_request(fake_engine, tmp_path):
    from prelude_b200.engine import cli
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(tiny.TINY_B))
    assert cli.main(["--model", str(folder), "--prompt-ids", "1", "--no-chunked-prefill", "--max-num-batched-tokens", "8"]) == 0
    assert fake_engine["kw"]["max_num_batched_tokens"] == tiny.TINY_B["max_position_embeddings"]
    assert cli.main(["--model", str(folder), "--prompt-ids", "1", "--chunked-prefill", "--max-num-batched-tokens", "8"]) == 0
    assert fake_engine["kw"]["max_num_batched_tokens"] == 8


def test_refusals(fake_engine, capsys):
    from prelude_b200.engine import cli
    assert cli.main(["--model", "m"]) == 2 and "at least one prompt" in capsys.readouterr().err
    assert cli.main(["--model", "m", "--prompt-ids", "1", "--device", "cpu"]) == 2 and "no cpu path" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        cli.main(["--model", "m", "--prompt-ids", "1", "--dtype", "fp8"])
