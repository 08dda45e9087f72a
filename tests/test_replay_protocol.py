"""The replay program's protocol on the host, with a stand-in for the model: which files are written, in which
order the rows come, what is printed after every step, what ends a request, and what a bad line gives."""
import json
import os

import numpy as np
import pytest
import torch


class _Cache:
    def __init__(self):
        self.live = set()

    def has_request(self, rid):
        return rid in self.live


class _Runner:
    """Logits row of a wanted place = [position of the token in its request, its token id, number of entries of the step]."""

    def __init__(self):
        self.cache, self.fed, self.finished, self.graphs = _Cache(), {}, [], False

    def enable_step_graphs(self):
        self.graphs = True

    def step(self, entries):
        rows = []
        for e in entries:
            base = self.fed.get(e.request_id, 0)
            self.cache.live.add(e.request_id)
            for w in e.want:
                rows.append([base + w, e.tokens[w], len(entries)])
            self.fed[e.request_id] = base + len(e.tokens)
        return torch.tensor(rows, dtype=torch.float32).reshape(len(rows), 3)

    def finish(self, rid):
        self.cache.live.discard(rid)
        self.fed.pop(rid, None)
        self.finished.append(rid)


@pytest.fixture
def fake(monkeypatch):
    from prelude_b200.engine import replay
    runner, made = _Runner(), {}
    monkeypatch.setattr(replay, "load_model", lambda folder, dtype, device: ("model", folder, dtype))
    monkeypatch.setattr(replay, "make_runner", lambda model, **kw: made.update(kw) or runner)
    return replay, runner, made


def test_steps_files_and_lines(fake, tmp_path):
    replay, runner, made = fake
    lines = [
        json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}),
        "",
        json.dumps({"step": 1, "entries": [{"id": "b", "tokens": [9, 8], "want": []}, {"id": "a", "tokens": [4], "want": [0]}], "end": []}),
        json.dumps({"step": 2, "entries": [{"id": "b", "tokens": [7, 6], "want": []}], "end": ["a"]}),
        json.dumps({"step": 7, "entries": [{"id": "b", "tokens": [1], "want": [0]}, {"id": "a", "tokens": [2, 3], "want": [1, 0]}], "end": ["a", "b", "never seen"]}),
        json.dumps({"step": 8, "entries": [], "end": []}),
    ]
    said = []
    n = replay.replay("folder", "float32", str(tmp_path / "out"), 200, lines, page_size=16, say=said.append)
    assert n == 5 and said == ["done 0", "done 1", "done 2", "done 7", "done 8"]
    assert made["num_pages"] == 13 and made["page_size"] == 16 and made["max_request_tokens"] == 200 and runner.graphs
    files = sorted(os.listdir(tmp_path / "out"))
    assert files == ["0.f32", "1.f32", "7.f32"]                    # nothing was wanted in steps 2 and 8
    read = lambda s: np.fromfile(tmp_path / "out" / f"{s}.f32", dtype="<f4").reshape(-1, 3).tolist()
    assert read(0) == [[0, 5, 1], [2, 3, 1]]
    assert read(1) == [[3, 4, 2]]                                  # a's fourth token, in the order of the entries
    assert read(7) == [[4, 1, 2], [1, 3, 2], [0, 2, 2]]            # a was ended and starts again at 0; want's own order
    assert runner.finished == ["a", "a", "b"]                      # a request that is not live is not finished again


@pytest.mark.parametrize("line", ["{not json", json.dumps({"entries": []}), json.dumps({"step": 0, "entries": [{"id": "a"}]}),
                                  json.dumps({"step": 0, "entries": [{"id": "a", "tokens": ["x"]}]})])
def test_a_bad_line_is_named(fake, tmp_path, line):
    replay, _, _ = fake
    with pytest.raises(ValueError, match="bad trace line"):
        replay.replay("folder", "float32", str(tmp_path / "out"), 64, [line], say=lambda s: None)


def test_command_line_refusals(capsys):
    from prelude_b200.engine import replay
    for bad in (["--page-size", "24"], ["--max-tokens", "0"]):
        args = ["--model", "m", "--dtype", "float32", "--out", "o", "--max-tokens", "64"] + bad
        with pytest.raises(SystemExit) as e:
            replay.main(args)
        assert e.value.code == 2
    with pytest.raises(SystemExit):
        replay.main(["--model", "m", "--dtype", "float16", "--out", "o", "--max-tokens", "64"])
