"""The engine against the plain implementation at the layer sizes that are benchmarked.

Random-weight models with the layer sizes of Qwen3-4B (2 of its 36 layers, the full vocabulary of 151,936),
Qwen3-8B (1 of 36 layers) and Qwen3-32B (1 of 64 layers; the last two with a vocabulary of 40,003, no power of
two and no multiple of eight), so that the kernels' paths for these widths run inside a model: pages with
permuted chunks, bulk-copy decode attention with its keys split over blocks and merged, the tcgen05 prompt
attention behind a cached prefix, the streaming product with the output head's 151,936 rows, the down
projection as four partial sums, the library product above 16 rows, the paired-block tcgen05 product with the
activation in its epilogue for a long prompt's gate/up projection.

Weights are drawn on the GPU and rounded to bfloat16 once; the 32-bit run, the bfloat16 run and the plain
implementation all use those same values, so no difference comes from the weights.

Tolerances.  32-bit: the yardstick is the plain implementation in float64.  The engine's 32-bit logits and the
plain 32-bit logits both differ from it by rounding alone; the engine is asked to stay within 1e-4 of the
float64 logits in absolute terms (logits here are of order 1), which is what the tiny configurations are held
to as well, and the plain 32-bit implementation's own distance from float64 is printed beside it.
bfloat16: within 3 % of the largest logit of the row, and within 2 % in the root-mean-square sense (measured:
1.0 to 1.5 % and 0.9 to 1.3 %, the same for every way of cutting: it is the rounding of activations to 8 bits).
"""
import math

import pytest
import torch

import harness
from plain.qwen3_plain import forward_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = {
    # name: (config, layers of the full model)
    "4b": (dict(vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=2,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, tie_word_embeddings=True), 36),
    "8b": (dict(vocab_size=40003, hidden_size=4096, intermediate_size=12288, num_hidden_layers=1,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, tie_word_embeddings=False), 36),
    "32b": (dict(vocab_size=40003, hidden_size=5120, intermediate_size=25600, num_hidden_layers=1,
                 num_attention_heads=64, num_key_value_heads=8, head_dim=128, tie_word_embeddings=False), 64),
}
COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", max_position_embeddings=4096, rope_theta=1000000.0,
              rms_norm_eps=1e-6, attention_bias=False, use_sliding_window=False, hidden_act="silu")
PAGE = 16


def _ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class _Sized:
    """One configuration: its weights (bfloat16 values) on the CPU in float64 for the yardstick, and models on the GPU."""

    def __init__(self, name):
        from prelude_b200.weights.random_init import random_tensors
        self.cfg = dict(COMMON, **SIZES[name][0])
        t = random_tensors(self.cfg, seed=5, std=0.02, norm_jitter=0.05, dtype=torch.bfloat16, device=DEV)
        self.tensors = t
        self.cpu = {k: v.cpu() for k, v in t.items()}
        self._models = {}
        self._w = {}

    def weights(self, dtype):
        if dtype not in self._w:
            self._w[dtype] = {k: v.to(dtype) for k, v in self.cpu.items()}
        return self._w[dtype]

    def model(self, dtype):
        if dtype not in self._models:
            from prelude_b200.config import load_model_config
            from prelude_b200.engine.loading import build_model
            from prelude_b200.weights.loader import WeightStore
            spec = load_model_config(self.cfg).to_model_spec()
            self._models[dtype] = build_model(spec, WeightStore.from_tensors(self.tensors), dtype, DEV)
        return self._models[dtype]


_cache = {}


def _sized(name):
    # one configuration at a time on the GPU and in host memory
    if name not in _cache:
        _cache.clear()
        torch.cuda.empty_cache()
        _cache[name] = _Sized(name)
    return _cache[name]


def _runner(model, num_pages, **kw):
    from prelude_b200.engine.loading import make_runner
    return make_runner(model, page_size=PAGE, num_pages=num_pages, max_slots=32, **kw)


def _schedules(reqs):
    """The four ways of cutting: whole, the last 32 one by one, portions that put 64, 128 and 512 tokens behind a
    cached prefix (and go down to two tokens), and up to four live requests mixed."""
    return {"whole": harness.whole(reqs), "tail_decode": harness.tail_decode(reqs),
            "portions": harness.portions(reqs, sizes=(40, 64, 128, 2, 512, 17, 3)),
            "mixed": harness.mixed(reqs, max_live=4, seed=3, decode_tail=5)}


def _check(got, ref, dtype, what):
    worst, worst_rms = 0.0, 0.0
    for (rid, pos), row in got.items():
        want = ref[rid][pos]
        diff = (row.double() - want).abs()
        if dtype == torch.float32:
            assert float(diff.max()) <= 1e-4, f"{what}: request {rid} position {pos}: {float(diff.max()):.3e} from the float64 logits"
            worst = max(worst, float(diff.max()))
        else:
            scale, rms = float(want.abs().max()), float(want.pow(2).mean().sqrt())
            assert float(diff.max()) <= 3e-2 * scale, f"{what}: request {rid} position {pos}: {float(diff.max()):.3e} > 3 % of {scale:.3f}"
            assert float(diff.pow(2).mean().sqrt()) <= 2e-2 * rms, f"{what}: request {rid} position {pos}: rms error above 2 %"
            worst, worst_rms = max(worst, float(diff.max()) / scale), max(worst_rms, float(diff.pow(2).mean().sqrt()) / rms)
    return worst, worst_rms


@pytest.mark.parametrize("name", ["4b", "8b", "32b"])
def test_every_way_of_cutting_at_real_layer_sizes(name, monkeypatch):
    from prelude_b200.ops import linear as LN
    pair_rows, pair = [], LN.gemm_pair
    monkeypatch.setattr(LN, "gemm_pair", lambda x, *a, **k: (pair_rows.append(x.shape[0]), pair(x, *a, **k))[1])
    s = _sized(name)
    V = s.cfg["vocab_size"]
    if name == "4b":
        lens = {"r300": 300, "r790": 790, "r70": 70, "r33": 33, "r140": 140}
    else:
        lens = {"r230": 230, "r45": 45, "r100": 100}
    reqs = {rid: _ids(n, V, 900 + n) for rid, n in lens.items()}
    w64 = s.weights(torch.float64)
    ref = {rid: forward_logits(s.cfg, w64, toks, dtype=torch.float64) for rid, toks in reqs.items()}
    w32 = s.weights(torch.float32)
    longest = max(reqs, key=lambda r: len(reqs[r]))
    plain32 = float((forward_logits(s.cfg, w32, reqs[longest]).double() - ref[longest]).abs().max())
    del s._w[torch.float32]
    scheds = _schedules(reqs)
    if name == "4b":        # a captured prompt step long enough for the paired-block product (and a two-token rest behind it)
        scheds["long_portions"] = harness.portions(reqs, sizes=(788, 2))
    total = sum(-(-len(t) // PAGE) for t in reqs.values())
    for dtype in (torch.float32, torch.bfloat16):
        model = s.model(dtype)
        for cut, schedule in scheds.items():
            num_pages = harness.peak_tokens(schedule, PAGE) // PAGE
            if cut == "mixed":
                assert num_pages < total                     # the pool forces pages to be used again
            runner = _runner(model, num_pages, max_request_tokens=1024 if cut != "whole" and cut != "tail_decode" else None)
            if cut in ("portions", "mixed", "long_portions"):
                runner.enable_step_graphs()                  # the captured prompt steps that the entry point uses
            calls = len(pair_rows)
            got = harness.run_schedule(runner, schedule)
            assert len(got) == sum(len(t) for t in reqs.values())
            if cut == "long_portions" and dtype == torch.bfloat16:
                assert len(pair_rows) > calls             # captured with the paired-block product inside
            worst = _check(got, ref, dtype, f"{name} {cut}")
            print(f"{name} {str(dtype)[6:]} {cut}: worst {worst[0]:.3e} (rms {worst[1]:.3e}); plain 32-bit is {plain32:.3e} from float64")
            runner.cache.check()
            assert runner.cache.used_pages() == 0
            del runner
        del s._models[dtype]
        torch.cuda.empty_cache()
    if name == "4b":        # the 790-token prompt's gate/up projection went through the paired-block tcgen05 kernel
        assert pair_rows and max(pair_rows) >= LN.PAIR_MIN_ROWS


def test_a_long_prompt_through_the_fused_products_and_decoding_behind_it(monkeypatch):
    """1,600 tokens in one step at Qwen3-4B sizes in bfloat16: the merged q/k/v projection with norm, rotation and
    cache write in its epilogue and the gate/up projection with its activation (both on the paired-block tcgen05
    kernel), then four tokens one by one that read the pages which that epilogue wrote; logits at the prompt's
    first, middle and last position and at every decoded one against the plain implementation in float64."""
    from prelude_b200.ops import linear as LN
    s = _sized("4b")
    V = s.cfg["vocab_size"]
    T, tail = 1600, 4
    assert T >= LN.PAIR_QKV_MIN_ROWS and LN.PREFILL_GEMM != "cublas"
    toks = _ids(T + tail, V, 4242)
    rows = [0, T // 2 - 1, T - 1] + list(range(T, T + tail))
    ref = forward_logits(s.cfg, s.weights(torch.float64), toks, dtype=torch.float64, rows=rows)
    schedule = [([("long", toks[:T], [0, T // 2 - 1, T - 1])], [])]
    schedule += [([("long", [toks[T + i]], [0])], ["long"] if i == tail - 1 else []) for i in range(tail)]
    runner = _runner(s.model(torch.bfloat16), harness.peak_tokens(schedule, PAGE) // PAGE)
    taken = []
    fused = LN.qkv_heads
    monkeypatch.setattr("prelude_b200.parts.attention.qkv_heads",
                        lambda x, *a, **k: (taken.append(x.shape[0]), fused(x, *a, **k))[1])
    got = harness.run_schedule(runner, schedule)
    assert T in taken
    worst = _check(got, {"long": {pos: ref[i] for i, pos in enumerate(rows)}}, torch.bfloat16, "4b long prompt")
    print(f"4b bfloat16 long prompt: worst {worst[0]:.3e} (rms {worst[1]:.3e})")
    runner.cache.check()
    assert runner.cache.used_pages() == 0


@pytest.mark.parametrize("batch", [1, 8, 17])
def test_captured_decode_steps_at_real_layer_sizes(batch):
    """The captured decode step and the queued runs of it, through ``Engine`` in bfloat16, at batch 1, 8 (streaming
    products) and 17 (the library product's side of the 16-row line), with contexts whose keys the decode kernel
    splits over blocks: the LOGITS of the captured steps against the plain implementation's, teacher-forced on the
    tokens the engine chose."""
    from prelude_b200 import Engine
    from prelude_b200.ops import attention as A
    s = _sized("4b")
    V = s.cfg["vocab_size"]
    new = 12
    prompts = [_ids(150 + 23 * (i % 5), V, 40 + i) for i in range(batch)]
    eng = Engine(s.model(torch.bfloat16), page_size=PAGE, num_pages=batch * 20 + 8, max_running_requests=32,
                 max_model_len=512, decode_burst=8)
    seen = {}                                              # (request, position) -> logits row of a captured step
    run_step, run_burst = eng._run_step, eng._run_burst

    def watching_step(items):
        out = run_step(items)
        if all(it.n_tokens == 1 and it.samples for it in items) and eng.graphs.graphs.get(len(items)) is not None:
            g = eng.graphs.get(len(items))
            for i, it in enumerate(items):
                seen[(it.seq.request_id, it.start)] = g.logits[i].float().cpu()
        return out

    def watching_burst(items, k):
        out = run_burst(items, k)
        g = eng.burst_graphs.get(len(items))
        for i, it in enumerate(items):                     # the logits of the run's last step are still there
            seen[(it.seq.request_id, it.start + len(out) - 1)] = g.logits[i].float().cpu()
        return out

    eng._run_step, eng._run_burst = watching_step, watching_burst
    res = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert eng.stats().graph_steps >= new - 2 and len(seen) >= 2 * batch
    splits, _ = A.decode_splits(batch, 8, 128, 512, torch.device(DEV))
    assert splits > 1 or batch > 8, "the contexts must be long enough for the decode kernel to split the keys"
    w32 = s.weights(torch.float32)
    ids = {r.request_id: p + r.token_ids for p, r in zip(prompts, res)}
    worst = 0.0
    for rid, toks in ids.items():
        rows = sorted(pos for (r, pos) in seen if r == rid)
        ref = forward_logits(s.cfg, w32, toks[:max(rows) + 1], rows=rows)
        for j, pos in enumerate(rows):
            got, want = seen[(rid, pos)].double(), ref[j].double()
            scale = float(want.abs().max())
            diff = float((got - want).abs().max())
            assert diff <= 3e-2 * scale, f"request {rid} position {pos}: {diff:.3e} > 3 % of {scale:.3f}"
            assert float((got - want).pow(2).mean().sqrt()) <= 2e-2 * float(want.pow(2).mean().sqrt())
            worst = max(worst, diff / scale)
            # the token the engine took from these logits is the plain implementation's best, or within rounding of it
            tok = toks[pos + 1]
            assert float(want.max() - want[tok]) <= 3e-2 * scale
    print(f"batch {batch}: {len(seen)} captured rows, worst {worst:.3e} of the largest logit, {splits} key splits")
    eng.cache.check()
    assert eng.cache.used_pages() == 0
