"""bin/trace_run as a user runs it: a child process fed steps on standard input,
``done <step>`` after each, logits files compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import harness
import tiny
from plain.qwen3_plain import forward_logits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_trace(folder, dtype, schedule, out_dir, max_tokens):
    proc = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
                             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            stderr=subprocess.PIPE, text=True)
    wanted = {}
    fed = {}
    for n, (entries, ended) in enumerate(schedule):
        rec = {"step": n, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want in entries], "end": ended}
        proc.stdin.write(json.dumps(rec) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()                 # the next step may come only after this
        assert line == f"done {n}", (line, proc.stderr.read() if proc.poll() is not None else "")
        keys = []
        for rid, toks, want in entries:
            keys += [(rid, fed.get(rid, 0) + w) for w in want]
            fed[rid] = fed.get(rid, 0) + len(toks)
        for rid in ended:
            fed.pop(rid, None)
        wanted[n] = keys
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0, proc.stderr.read()
    return wanted


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "C", "E"])
def test_trace_run_mixed_with_reused_pages(tmp_path, which, dtype):
    cfg = tiny.PARAMS[which][0]
    folder = tiny.make_folder(tmp_path, which, torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs = {f"r{i}": tiny.random_ids(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([70, 45, 33, 100, 64, 20])}
    schedule = harness.mixed(reqs, max_live=4, seed=3)
    # some steps want nothing at all, some only their last place
    schedule = [([(rid, toks, [] if (n % 5 == 1) else ([len(toks) - 1] if n % 5 == 2 else want))
                  for rid, toks, want in entries], ended) for n, (entries, ended) in enumerate(schedule)]
    max_tokens = harness.peak_tokens(schedule, 64)            # each request rounded up to a multiple of 64
    assert max_tokens < sum(-(-len(t) // 64) * 64 for t in reqs.values())
    out = str(tmp_path / "out")
    wanted = _run_trace(folder, dtype, schedule, out, max_tokens)
    w = tiny.read_weights(folder)
    ref = {rid: forward_logits(cfg, w, toks) for rid, toks in reqs.items()}
    atol, rel = (1e-4, 0.0) if dtype == "float32" else (0.0, 3e-2)
    checked = 0
    for n, keys in wanted.items():
        path = os.path.join(out, f"{n}.f32")
        if not keys:
            assert not os.path.exists(path)
            continue
        got = np.fromfile(path, dtype="<f4").reshape(len(keys), cfg["vocab_size"])
        for row, (rid, pos) in zip(got, keys):
            want = ref[rid][pos].numpy()
            assert np.abs(row - want).max() <= atol + rel * np.abs(want).max(), (n, rid, pos)
            checked += 1
    assert checked > 100


def test_trace_run_reports_errors_and_exits_nonzero(tmp_path):
    folder = tiny.make_folder(tmp_path, "A")
    run = lambda args, text: subprocess.run([os.path.join(ROOT, "bin", "trace_run")] + args, input=text,  # noqa: E731
                                            capture_output=True, text=True, timeout=600)
    base = ["--model", folder, "--dtype", "float32", "--out", str(tmp_path / "o")]
    r = run(base + ["--max-tokens", "64"], json.dumps({"step": 0, "entries": [{"id": "a", "tokens": list(range(100)), "want": []}], "end": []}) + "\n")
    assert r.returncode != 0 and "OutOfPages" in r.stderr
    r = run(base + ["--max-tokens", "64"], json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [999], "want": [0]}], "end": []}) + "\n")
    assert r.returncode != 0 and "token ids" in r.stderr
    r = run(base + ["--max-tokens", "64"], "")
    assert r.returncode == 0 and r.stdout == ""
    r = run(["--model", str(tmp_path / "nowhere"), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"], "")
    assert r.returncode != 0 and "config.json" in r.stderr
