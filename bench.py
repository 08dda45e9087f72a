"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--layers L] [--impl ours|reference]

The default run has the layer sizes of Qwen3-4B (BASELINE.json configs[2]) with
random weights in bfloat16, a batch of 8 requests that each hold a 2,048-token
prefix in a cache laid out for 4,096-token contexts with 16-token pages, and
prints one JSON line:

  value     decoded tokens a second, timed on the device: K replays of the captured
            decode step (model + sampling, the sampled token fed back on the device)
            between two CUDA events;
  e2e       the same through Engine.generate(): host token ids in, host token ids
            out, every step's inputs copied from pinned memory and its tokens read back;
  prefill   one 2,048-token prompt through the step function;
  roofline  the bytes a decode step has to read (every weight once, the cache of
            the live requests) over its time, against the measured copy bandwidth;
  points    the device-timed value at batch 1 and 64.

Every decode step reads the whole model (8 GB at full size), far more than the
126 MB L2, so no flush is needed between steps ("l2": "inputs_exceed_l2").

``--workload serving`` measures something else and prints a line of its own: a
mixed continuous batch through Engine.generate() (BASELINE.json configs[3]: 32
requests, prompts of 128 to 2,048 tokens cut into portions of 512 beside the
running decodes, 256 tokens each), as generated tokens a second by the wall clock.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=2560,
                intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=True, attention_bias=False, use_sliding_window=False, hidden_act="silu")
# the layer sizes of the other two Qwen3 dense models, for --model-size (the default run is the 4B model)
OTHER_SIZES = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
}
CONTEXT_LEN, PREFIX_LEN, PAGE_SIZE, PREFILL_TOKENS = 4096, 2048, 16, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = dict(FALLBACK_PEAKS, source="measured")
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            v = raw.get(k)
            if isinstance(v, dict):                          # a record around the figure
                v = v.get("value")
            if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                out[k] = float(v)
        return out
    except (OSError, ValueError, AttributeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [p.strip() for p in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        rows = [p for t, p in self.samples if any(a <= t <= b for a, b in windows) and len(p) >= 6]
        if not rows:
            rows = [p for _, p in self.samples if len(p) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = [int(float(p[0])) for p in rows if p[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for p in rows for n, v in zip(names, p[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": int(float(rows[0][1])) if rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


MODEL = QWEN3_4B            # what --model-size chose


def build_engine(layers, max_running, num_pages, prefill_chunk=0):
    import torch
    from prelude_b200 import Engine
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model
    from prelude_b200.weights.loader import WeightStore
    from prelude_b200.weights.random_init import random_tensors
    cfg = dict(MODEL, num_hidden_layers=layers)
    tensors = random_tensors(cfg, seed=0, std=0.02, norm_jitter=0.05, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(load_model_config(cfg).to_model_spec(), WeightStore.from_tensors(tensors), "bf16", "cuda:0")
    del tensors
    torch.cuda.empty_cache()
    return Engine(model, page_size=PAGE_SIZE, num_pages=num_pages, max_running_requests=max_running,
                  max_num_batched_tokens=max(8192, PREFILL_TOKENS), long_prefill_token_threshold=prefill_chunk,
                  max_model_len=CONTEXT_LEN, cuda_graph=True, cuda_graph_max_bs=64), cfg


def weight_bytes_per_step(cfg):
    """Bytes of weights one decode step reads: every matrix once (the tied
    embedding table once, as the output head), norm scales in float32."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    per_layer = 2 * (qkv * H + H * cfg["num_attention_heads"] * cfg["head_dim"] + 3 * I * H) + 4 * (2 * H + 2 * cfg["head_dim"])
    head = 2 * cfg["vocab_size"] * H          # tied or not: the head once; a separate table only at the step's token rows
    return L * per_layer + head + 4 * H


def kv_bytes_per_token(cfg):
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, T):
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nH, D = cfg["num_attention_heads"], cfg["head_dim"]
    qkv = (nH + 2 * cfg["num_key_value_heads"]) * D
    gemm = 2 * T * L * (qkv * H + H * nH * D + 3 * I * H) + 2 * 1 * cfg["vocab_size"] * H
    attn = L * 4 * nH * D * (T * (T + 1) // 2)          # QK^T and PV over the causal half
    return gemm + attn


def time_decode(engine, cfg, batch, steps, warmup, seed):
    """Device time of ``steps`` decode steps at ``batch`` requests with PREFIX_LEN-token prefixes."""
    import torch
    from prelude_b200.engine.graph import DecodeGraph
    from prelude_b200.engine.runner import StepEntry
    from prelude_b200.ops import library
    runner, cache = engine.runner, engine.cache
    g = torch.Generator().manual_seed(seed)
    rids = [f"bench{seed}_{i}" for i in range(batch)]
    for rid in rids:                                     # real prefill fills the cache
        ids = torch.randint(0, cfg["vocab_size"], (PREFIX_LEN,), generator=g).tolist()
        runner.step([StepEntry(rid, ids, [])], check_status=False)
    total = PREFIX_LEN + warmup + steps + 1
    for rid in rids:                                     # room for every token the loop will write
        cache.grow(rid, total)
    cache.flush_table_updates()
    graph = DecodeGraph(runner, batch, self_feeding=True)
    tokens = torch.randint(0, cfg["vocab_size"], (batch,), generator=g).tolist()
    graph.load(tokens, [PREFIX_LEN] * batch, [cache.slot_of(r) for r in rids], [0.0] * batch, [0] * batch, [0] * batch)
    graph.capture()
    graph.load(tokens, [PREFIX_LEN] * batch, [cache.slot_of(r) for r in rids], [0.0] * batch, [0] * batch, [0] * batch)
    for _ in range(warmup):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.time()
    start.record()
    torch.cuda.nvtx.range_push("timed_decode")          # lets a profiler pick these launches out
    for _ in range(steps):
        graph.replay()
    torch.cuda.nvtx.range_pop()
    end.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = start.elapsed_time(end)
    status = int(graph.status.item())
    if status != 0:
        raise RuntimeError(f"decode loop raised kernel status {status}")
    if TIMELINE:
        print_timeline(graph)
    for rid in rids:
        runner.finish(rid)
    del graph
    avg_ctx = PREFIX_LEN + warmup + (steps + 1) / 2.0
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches_per_step": None,
            "avg_ctx": avg_ctx, "window": (t0, t1)}, library


TIMELINE = False


def print_timeline(graph):
    """One more replay of the captured step with the kernels' timeline marks on (a library built with
    PRELUDE_TIMELINE=1): for every kernel of the step's second layer, when its first block started, when the kernel
    before it had finished, when its input had arrived and when its first and last block were done, in
    microseconds from the layer's first mark."""
    import torch
    from prelude_b200.ops import timeline
    timeline.enable()
    timeline.reset()
    graph.replay()
    torch.cuda.synchronize()
    marks = timeline.read()
    # a layer begins with the add+norm that precedes the qkv product: cut the step at every second norm entry
    starts = [i for i, m in enumerate(marks) if m.kernel == "add_rmsnorm" and m.mark == "entry" and not m.last_block]
    if len(starts) < 5:
        print(f"timeline: {len(marks)} marks, too few to show a layer", file=sys.stderr)
        return
    lo, hi = starts[2], starts[4]                           # the second layer's two norms and what lies between
    t0 = marks[lo].ns
    print("timeline of one layer of the captured decode step (us from the layer's first mark):", file=sys.stderr)
    for m in marks[lo:hi]:
        print(f"  {(m.ns - t0) / 1e3:8.2f}  {m.kernel:22s} {m.mark:10s} {'last block' if m.last_block else 'first block'}", file=sys.stderr)
    print(f"  {(marks[hi].ns - t0) / 1e3:8.2f}  next layer begins", file=sys.stderr)


def time_prefill(engine, cfg, warmup, reps=3):
    import torch
    from prelude_b200.engine.runner import StepEntry
    runner = engine.runner
    g = torch.Generator().manual_seed(7)
    times = []
    t0 = time.time()
    for i in range(warmup + reps):
        ids = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        if i >= warmup:
            torch.cuda.nvtx.range_push("timed_prefill")
        runner.step([StepEntry(f"prefill{i}", ids, [PREFILL_TOKENS - 1])], check_status=False)
        if i >= warmup:
            torch.cuda.nvtx.range_pop()
        e.record()
        torch.cuda.synchronize()
        runner.finish(f"prefill{i}")
        if i >= warmup:
            times.append(s.elapsed_time(e))
    return min(times), (t0, time.time())


def time_e2e(engine, cfg, batch, steps):
    """Decoded tokens a second through Engine.generate(): after each request's first token."""
    import torch
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab_size"], (PREFIX_LEN,), generator=g).tolist() for _ in range(batch)]
    # warm up outside the timed call: the decode step is captured per batch size at its first use, and
    # requests that finish a step apart leave smaller batches behind
    engine.warmup(range(1, batch + 1))
    engine.generate([p[:32] for p in prompts], temperature=0.0, max_new_tokens=4, ignore_eos=True)
    import copy
    before = copy.copy(engine.stats())
    t0 = time.time()
    res = engine.generate(prompts, temperature=0.0, max_new_tokens=steps + 1, ignore_eos=True)
    t1 = time.time()
    decode_ms = max(r.total_ms for r in res) - max(r.ttft_ms for r in res)
    toks = sum(r.completion_tokens - 1 for r in res)
    # bytes that the timed call copied, counted by the engine from the tensors it copied, over the steps it ran
    # (a run of queued decode steps loads its inputs once and reads every step's tokens back)
    st = engine.stats()
    n_steps = max(1, st.steps - before.steps)
    return {"value": toks / (decode_ms / 1e3), "unit": "tok/s",
            "h2d_bytes_per_step": round((st.h2d_bytes - before.h2d_bytes) / n_steps, 1),
            "d2h_bytes_per_step": round((st.d2h_bytes - before.d2h_bytes) / n_steps, 1), "decode_ms": decode_ms}, (t0, t1)


def serve(args):
    """A mixed continuous batch through ``Engine.generate`` (host tokens in, host tokens out): ``--requests`` prompts
    of uniform random ids with lengths uniform in [128, 2048], prompts cut into portions of ``--prefill-chunk``
    tokens beside the running decodes, ``--new-tokens`` greedy tokens each.  One JSON line of its own."""
    import copy
    import random
    import time
    import torch
    rng = random.Random(7)
    lens = [rng.randint(128, 2048) for _ in range(args.requests)]
    pages = sum(-(-(n + args.new_tokens + 1) // PAGE_SIZE) for n in lens) + 64
    engine, cfg = build_engine(args.layers, args.requests, pages, prefill_chunk=args.prefill_chunk)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    engine.warmup(range(1, args.requests + 1))
    engine.warmup_prompt_steps([args.prefill_chunk])
    engine.generate(prompts[:2], temperature=0.0, max_new_tokens=4, ignore_eos=True)
    before = copy.copy(engine.stats())
    torch.cuda.synchronize()
    clocks = ClockSampler()
    clocks.start()
    t0 = time.time()
    results = engine.generate(prompts, temperature=0.0, max_new_tokens=args.new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    t1 = time.time()
    clocks.stop()
    st = engine.stats()
    out_tokens = sum(r.completion_tokens for r in results)
    ttft = sorted(r.ttft_ms for r in results)
    line = {
        "metric": f"serving: {args.requests} requests, prompts of 128 to 2,048 tokens in portions of {args.prefill_chunk}, "
                  f"{args.new_tokens} greedy tokens each (Qwen3-{args.model_size.upper()} sizes, random weights, bf16)",
        "value": round(out_tokens / (t1 - t0), 1), "unit": "generated tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": "ours", "seconds": round(t1 - t0, 3),
        "prompt_tokens": sum(lens), "generated_tokens": out_tokens,
        "total_tok_s": round((sum(lens) + out_tokens) / (t1 - t0), 1),
        "ttft_ms": {"p50": round(statistics.median(ttft), 1), "p95": round(ttft[int(0.95 * (len(ttft) - 1))], 1), "max": round(ttft[-1], 1)},
        "steps": st.steps - before.steps, "decode_steps": st.decode_steps - before.decode_steps,
        "captured_steps": st.graph_steps - before.graph_steps, "preemptions": st.preemptions - before.preemptions,
        "config": {"model": f"qwen3-{args.model_size}-sizes", "layers": args.layers, "layers_full": MODEL["num_hidden_layers"],
                   "requests": args.requests, "prefill_chunk": args.prefill_chunk, "new_tokens": args.new_tokens, "page_size": PAGE_SIZE},
        "clocks": clocks.summary([(t0, t1)]),
    }
    print(json.dumps(line))
    return 0


def main():
    global MODEL, PREFIX_LEN, CONTEXT_LEN, PAGE_SIZE, PREFILL_TOKENS, TIMELINE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--model-size", default="4b", choices=["4b", "8b", "32b"],
                    help="layer sizes of another Qwen3 dense model (the headline run is 4b)")
    ap.add_argument("--prefix-len", type=int, default=PREFIX_LEN, help="tokens every request holds before the timed decode steps")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt (the contract's is 2,048)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per page of the key/value cache")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels' timeline of one layer of the decode step to stderr (needs PRELUDE_TIMELINE=1 in the environment)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="serving: a mixed continuous batch through Engine.generate instead of the decode step (a line of its own)")
    ap.add_argument("--requests", type=int, default=32, help="serving: number of requests")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="serving: tokens per portion of a prompt")
    ap.add_argument("--new-tokens", type=int, default=256, help="serving: generated tokens per request")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip install of the reference fails (not installable: neither setup.py nor pyproject.toml; a Rust workspace with git-only "
                          "dependencies, no cargo or rustc and no network here)"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus N with N > 1 is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    TIMELINE = args.timeline
    if args.model_size != "4b":
        MODEL = dict(QWEN3_4B, **OTHER_SIZES[args.model_size])
    PREFIX_LEN = args.prefix_len
    PAGE_SIZE = args.page_size
    PREFILL_TOKENS = args.prefill_tokens
    CONTEXT_LEN = max(CONTEXT_LEN, PREFIX_LEN + args.steps + args.warmup + 64, PREFILL_TOKENS + 64)
    args.layers = args.layers or MODEL["num_hidden_layers"]
    if args.workload == "serving":
        CONTEXT_LEN = max(CONTEXT_LEN, 2048 + args.new_tokens + 64)
        return serve(args)
    import torch
    pk = peaks()
    # cache: the largest point (64 requests) with room for prefix + generated tokens, in whole pages
    biggest = 64 if not args.no_points else args.batch
    pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
    num_pages = max(biggest, args.batch) * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8
    engine, cfg = build_engine(args.layers, max(64, args.batch) + 2, num_pages)
    clocks = ClockSampler()
    clocks.start()
    windows = []

    prefill_ms, w = time_prefill(engine, cfg, args.warmup)
    windows.append(w)
    dec, library = time_decode(engine, cfg, args.batch, args.steps, args.warmup, seed=1)
    windows.append(dec["window"])
    points = {}
    if not args.no_points:
        for b, k in ((1, min(args.steps, 128)), (64, min(args.steps, 64))):
            if b == args.batch:
                points[f"decode_b{b}"] = round(dec["tok_s"], 1)
                continue
            d, _ = time_decode(engine, cfg, b, k, args.warmup, seed=100 + b)
            windows.append(d["window"])
            points[f"decode_b{b}"] = round(d["tok_s"], 1)
    e2e, w = time_e2e(engine, cfg, args.batch, args.steps)
    windows.append(w)
    clocks.stop()

    launches_per_step = engine.graphs.get(args.batch).launches
    step_bytes = weight_bytes_per_step(cfg) + args.batch * dec["avg_ctx"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    pf = prefill_flops(cfg, PREFILL_TOKENS)
    line = {
        "metric": f"decode tok/s (Qwen3-{args.model_size.upper()} sizes, random weights, bf16, batch {args.batch}, "
                  f"{PREFIX_LEN:,}-token prefixes)",
        "value": round(dec["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"qwen3-{args.model_size}-sizes", "layers": args.layers, "layers_full": MODEL["num_hidden_layers"],
                   "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
                   "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"], "tie_word_embeddings": cfg["tie_word_embeddings"],
                   "global_batch": args.batch, "seq_len": PREFIX_LEN, "context_len": CONTEXT_LEN,
                   "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single",
                   "l2": "inputs_exceed_l2", "peaks": pk["source"]},
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items() if k != "decode_ms"},
        "gpu_launches": int(launches_per_step * args.steps),
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
