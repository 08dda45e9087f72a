"""Parts from outside the package, and cache groups with a window, through the entry point with captured steps
switched on: a mixer with state of its own and a routed feed-forward that decide on the host (the engine then
launches their steps), a routed feed-forward without host decisions (its steps are captured), an embedding and a
head of another kind, and a layer that keeps a window of its keys."""
import math
from dataclasses import dataclass, replace

import pytest
import torch

import tiny
from plain import qwen3_plain as plain
from test_gpu_parts import (DecaySpec, RoutedSpec, LinearAngleSpec, _plain_routed_and_linear_angle, _plain_toy,
                            _register_toy, _register_toy_ff_and_position, _store)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _greedy(logits_of, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(logits_of(ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out


def _engine(model, page, **kw):
    from prelude_b200 import Engine
    args = dict(page_size=page, num_pages=64, max_running_requests=4, max_num_batched_tokens=16)
    args.update(kw)
    return Engine(model, **args)


def test_parts_that_decide_on_the_host_run_launched_and_capturable_ones_captured():
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model
    from prelude_b200.ops.linear import linear
    from prelude_b200.parts.registry import register_part, unregister_part
    from prelude_b200.weights.loader import TensorReq
    from prelude_b200.weights.random_init import random_tensors
    Decay = _register_toy()
    Decay.capturable = False                      # it loops over requests on the host
    _register_toy_ff_and_position()

    @register_part("feed_forward", "toy_routed_dense")
    class RoutedDense:
        """The routed feed-forward without a decision on the host: every expert runs on every token and the
        router's choice masks the results, so the step has the same launches whatever the tokens are."""

        def __init__(self, spec, prefix):
            self.spec, self.prefix = spec, prefix

        def tensors(self):
            s, p = self.spec, self.prefix
            out = {f"{p}.router.weight": TensorReq((s.n_experts, s.hidden_size))}
            for e in range(s.n_experts):
                out[f"{p}.experts.{e}.up.weight"] = TensorReq((s.expert_size, s.hidden_size))
                out[f"{p}.experts.{e}.down.weight"] = TensorReq((s.hidden_size, s.expert_size))
            return out

        def load(self, get, ctx):
            s, p = self.spec, self.prefix
            self.router = get(f"{p}.router.weight").to(ctx.device, torch.float32)
            self.up = [get(f"{p}.experts.{e}.up.weight").to(ctx.device, ctx.dtype).contiguous() for e in range(s.n_experts)]
            self.down = [get(f"{p}.experts.{e}.down.weight").to(ctx.device, ctx.dtype).contiguous() for e in range(s.n_experts)]

        def forward(self, x):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            choice = probs.argmax(dim=-1, keepdim=True)
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.spec.n_experts):
                y = linear(torch.relu(linear(x, self.up[e])), self.down[e]).float() * probs[:, e:e + 1]
                out += torch.where(choice == e, y, torch.zeros_like(y))
            return out.to(x.dtype)

    try:
        cfg, init, page = tiny.PARAMS["A"]
        H, D, E, I = cfg["hidden_size"], cfg["head_dim"], 3, 40
        base = load_model_config(cfg).to_model_spec()
        b0, b1 = base.blocks
        prompts = [tiny.random_ids(n, cfg["vocab_size"], 60 + n) for n in (21, 6, 33)]
        new = 14

        # (1) a mixer with state, looping on the host: not capturable, so the engine launches its steps
        spec = replace(base, blocks=(b0, replace(b1, mixer=DecaySpec(H, 0.9))))
        w = {k: v for k, v in random_tensors(cfg, **init).items() if not k.startswith("model.layers.1.self_attn.")}
        w["model.layers.1.self_attn.mix.weight"] = torch.randn(H, H, generator=torch.Generator().manual_seed(2)) * 0.1
        model = build_model(spec, _store(w), torch.float32, DEV)
        caps = model.runtime_caps()
        assert caps.state_slots and caps.kv_cache and not caps.cuda_graph
        eng = _engine(model, page, cuda_graph=True)
        assert eng.graphs is None and eng.runner.step_graphs is None
        got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
        want = [_greedy(lambda ids: _plain_toy(cfg, w, ids, 0.9), p, new) for p in prompts]
        assert [r.token_ids for r in got] == want
        eng.cache.check()
        assert eng.cache.used_pages() == 0

        # (2) the routed feed-forward: the one that picks rows on the host (launched), the dense one (captured)
        pos = LinearAngleSpec(D, D // 2, 0.07, cfg["max_position_embeddings"])
        g = torch.Generator().manual_seed(5)
        w = {k: v for k, v in random_tensors(cfg, **init).items() if not k.startswith("model.layers.1.mlp.")}
        w["model.layers.1.mlp.router.weight"] = torch.randn(E, H, generator=g)
        for e in range(E):
            w[f"model.layers.1.mlp.experts.{e}.up.weight"] = torch.randn(I, H, generator=g) * 0.1
            w[f"model.layers.1.mlp.experts.{e}.down.weight"] = torch.randn(H, I, generator=g) * 0.1
        want = [_greedy(lambda ids: _plain_routed_and_linear_angle(cfg, w, ids, E, D // 2, 0.07), p, new) for p in prompts]
        from prelude_b200.parts.registry import part_class
        part_class("feed_forward", "toy_routed").capturable = False
        for kind, captured in (("toy_routed", False), ("toy_routed_dense", True)):
            spec = replace(base, blocks=(replace(b0, mixer=replace(b0.mixer, position=pos)),
                                         replace(b1, mixer=replace(b1.mixer, position=pos),
                                                 feed_forward=RoutedSpec(H, I, E, kind=kind))))
            model = build_model(spec, _store(w), torch.float32, DEV)
            assert model.runtime_caps().cuda_graph == captured
            eng = _engine(model, page, cuda_graph=True, decode_burst=4)
            got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
            assert [r.token_ids for r in got] == want, kind
            assert (eng.stats().graph_steps > 0) == captured
            if captured:
                assert eng.runner.graph_steps_run > 0          # prompt steps were replayed from their pieces too
            eng.cache.check()
            assert eng.cache.used_pages() == 0
    finally:
        for fam, kind in (("mixer", "toy_decay"), ("feed_forward", "toy_routed"), ("feed_forward", "toy_routed_dense"),
                          ("position", "toy_linear_angle")):
            unregister_part(fam, kind)


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    name: str = "model.embed_tokens.weight"
    kind: str = "toy_scaled_embedding"


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    hidden_size: int
    cap: float
    name: str = "lm_head.weight"
    kind: str = "toy_capped_head"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_an_embedding_and_a_head_of_another_kind_are_registrations(dtype):
    """A scaled embedding and a head whose logits are capped (cap * tanh(logits / cap)), defined here: chosen by
    ``ModelSpec.embedding`` / ``ModelSpec.head``, nothing in the package changes."""
    import harness
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model, make_runner
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.linear import linear
    from prelude_b200.parts.registry import register_part, unregister_part
    from prelude_b200.weights.loader import TensorReq
    from prelude_b200.weights.random_init import random_tensors

    @register_part("embedding", "toy_scaled_embedding")
    class ScaledEmbedding:
        def __init__(self, spec, prefix=""):
            self.spec = spec

        def tensors(self):
            return {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}

        def load(self, get, ctx):
            self.table = get(self.spec.name).to(ctx.device, ctx.dtype).contiguous()

        def forward(self, batch):
            return K.embed_gather(batch.token_ids, self.table) * self.spec.scale

    @register_part("head", "toy_capped_head")
    class CappedHead:
        def __init__(self, spec, prefix=""):
            self.spec = spec

        def tensors(self):
            return {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}, {}

        def load(self, get, ctx, embedding):
            self.weight = get(self.spec.name).to(ctx.device, ctx.dtype).contiguous()

        def forward(self, x):
            return self.spec.cap * torch.tanh(linear(x, self.weight, None, out_dtype=torch.float32) / self.spec.cap)

    try:
        cfg, init, page = tiny.PARAMS["B"]                          # a head of its own
        V, H = cfg["vocab_size"], cfg["hidden_size"]
        scale, cap = math.sqrt(H), 0.5
        w = {k: v.to(dtype) for k, v in random_tensors(cfg, **init).items()}
        spec = replace(load_model_config(cfg).to_model_spec(), embedding=ScaledEmbeddingSpec(V, H, scale),
                       head=CappedHeadSpec(V, H, cap))
        wf = {k: v.float() for k, v in w.items()}
        wf["model.embed_tokens.weight"] = wf["model.embed_tokens.weight"] * scale
        reqs = {"x": tiny.random_ids(37, V, 1), "y": tiny.random_ids(12, V, 2)}
        ref = {rid: cap * torch.tanh(plain.forward_logits(cfg, wf, toks) / cap) for rid, toks in reqs.items()}
        plain_ref = plain.forward_logits(cfg, {k: v.float() for k, v in w.items()}, reqs["x"])
        assert (ref["x"] - plain_ref).abs().max() > 1e-2            # both ends matter
        model = build_model(spec, _store(w), dtype, DEV)
        for cut in (harness.whole, harness.portions, harness.mixed):
            schedule = cut(reqs)
            runner = make_runner(model, page_size=page, num_pages=harness.peak_tokens(schedule, page) // page, max_slots=4)
            for (rid, pos), row in harness.run_schedule(runner, schedule).items():
                want = ref[rid][pos]
                assert (row - want).abs().max() <= (1e-4 if dtype == torch.float32 else 3e-2 * float(want.abs().max()))
    finally:
        unregister_part("embedding", "toy_scaled_embedding")
        unregister_part("head", "toy_capped_head")


@pytest.mark.parametrize("graphs,burst,chunk", [(False, 1, 0), (True, 1, 5), (True, 6, 7)])
def test_a_layer_with_a_window_through_the_entry_point(graphs, burst, chunk):
    """A window shorter than what is generated, pages shorter than the window: pages that the window has passed go
    back while the request runs (their entries in the device-resident tables turn to -1), prompt portions cross the
    window's edge, captured steps and queued runs of them read the trimmed tables.  32-bit, so the tokens are the
    plain implementation's."""
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model
    from prelude_b200.weights.random_init import random_tensors
    cfg, init, page = tiny.PARAMS["A"]
    window = 9
    w = random_tensors(cfg, seed=5, std=0.08, norm_jitter=0.3)
    spec = load_model_config(cfg).to_model_spec()
    b0, b1 = spec.blocks
    spec = replace(spec, blocks=(b0, replace(b1, mixer=replace(b1.mixer, window=window))))
    prompts = [tiny.random_ids(n, cfg["vocab_size"], 80 + n) for n in (30, 7, 19)]
    new = 25
    wf = {k: v.float() for k, v in w.items()}
    want = [_greedy(lambda ids: plain.forward_logits(cfg, wf, ids, windows={1: window}), p, new) for p in prompts]
    full = _greedy(lambda ids: plain.forward_logits(cfg, wf, ids), prompts[0], new)
    assert full != want[0]                                          # the window changes what is generated
    model = build_model(spec, _store(w), torch.float32, DEV)
    eng = _engine(model, page, cuda_graph=graphs, decode_burst=burst, long_prefill_token_threshold=chunk, num_pages=40)
    assert len(eng.cache.groups) == 2
    windowed = next(g for g in eng.cache.groups if g.need.window == window)
    peak = {"all": 0, "window": 0}
    step_once = eng.step_once

    def watching():
        out = step_once()
        peak["window"] = max(peak["window"], windowed.allocator.num_used)
        peak["all"] = max(peak["all"], eng.cache.used_pages())
        eng.cache.check()
        return out

    eng.step_once = watching
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    # three requests of up to 55 tokens: 14 pages each without a window; with it, 3 or 4 (a run of queued steps holds its pages until it ends)
    assert peak["all"] >= 30 and peak["window"] <= 3 * (4 + (burst + 3) // 4)
    if graphs:
        assert eng.stats().graph_steps > 0
    assert eng.cache.used_pages() == 0 and not eng.cache.requests


def test_a_status_word_raised_in_a_captured_step_fails_that_step_only():
    """A captured step whose status word comes back non-zero raises; the next call on the same engine (and the same
    captured step) starts with a clear word and gives the right tokens."""
    from prelude_b200 import Engine
    from prelude_b200.engine.batch import StepError
    from prelude_b200.engine.graph import DecodeGraph
    import tempfile
    cfg = tiny.PARAMS["A"][0]
    with tempfile.TemporaryDirectory() as d:
        folder = tiny.make_folder(d, "A", torch.float32)
        w = tiny.read_weights(folder)
        eng = Engine(folder, dtype="f32", page_size=4, num_pages=32, max_running_requests=4, decode_burst=1)
        prompts = [tiny.random_ids(n, cfg["vocab_size"], 5 + n) for n in (9, 4)]
        want = [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
        assert [r.token_ids for r in eng.generate(prompts, temperature=0.0, max_new_tokens=8, ignore_eos=True)] == want
        replay, calls = DecodeGraph.replay, []

        def raising(self):
            replay(self)
            calls.append(1)
            if len(calls) == 2:
                self.status.fill_(12)                               # as if a product had given up a wait
        DecodeGraph.replay = raising
        try:
            with pytest.raises(StepError, match="code 12"):
                eng.generate(prompts, temperature=0.0, max_new_tokens=8, ignore_eos=True)
        finally:
            DecodeGraph.replay = replay
        eng.cache.check()
        assert eng.cache.used_pages() == 0 and not eng.has_work()
        assert [r.token_ids for r in eng.generate(prompts, temperature=0.0, max_new_tokens=8, ignore_eos=True)] == want
