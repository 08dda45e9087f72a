"""bench.py without a GPU: the roofline arithmetic against figures worked out by hand from the layer sizes, the
answer to more than one GPU, the reference arm's line, and the peaks file."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_bytes_and_flops_of_the_headline_configuration():
    import bench
    cfg = dict(bench.QWEN3_4B)
    H, I, L, V = 2560, 9728, 36, 151936
    per_layer = 2 * (6144 * H + H * 4096 + 3 * I * H)            # qkv, o, gate, up, down in bfloat16
    assert per_layer == 201_850_880
    norms = 4 * (2 * H + 2 * 128)                                 # two norms and the q/k norms of a layer, float32
    assert bench.weight_bytes_per_step(cfg) == L * (per_layer + norms) + 2 * V * H + 4 * H
    assert abs(bench.weight_bytes_per_step(cfg) - 8.045e9) < 0.005e9
    assert bench.kv_bytes_per_token(cfg) == 147_456               # 36 layers x 8 heads x 128 x (k, v) x 2 bytes
    flops = bench.prefill_flops(cfg, 2048)
    assert abs(flops - 16.12e12) < 0.02e12                        # 14.88 TFLOP of products + 1.24 TFLOP of attention
    # an untied model reads its head once a step as well; its table only at the rows of the step's tokens
    cfg32 = dict(bench.QWEN3_4B, **bench.OTHER_SIZES["32b"])
    assert abs(bench.weight_bytes_per_step(cfg32) - 63.97e9) < 0.2e9
    assert bench.kv_bytes_per_token(cfg32) == 262_144


def test_more_than_one_gpu_is_refused_with_one_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 2 and len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout


def test_reference_arm_says_why_it_is_unavailable():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "\n" not in line["unavailable"] and len(line["unavailable"]) > 20


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks()["source"] == "fallback" and bench.peaks()["hbm_gbs"] == 6650.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000.0, "bf16_tflops": 1500.0}))
    pk = bench.peaks()
    assert pk["source"] == "measured" and pk["hbm_gbs"] == 7000.0 and pk["bf16_tflops"] == 1500.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": {"value": 6900.0, "sm_mhz": 1965}, "bf16_tflops": -1}))
    pk = bench.peaks()
    assert pk["hbm_gbs"] == 6900.0 and pk["bf16_tflops"] == 1590.0       # a record around the figure; a figure that cannot be
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps([1, 2]))
    assert bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.peaks()["source"] == "fallback"
