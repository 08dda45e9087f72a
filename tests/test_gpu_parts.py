"""Each part alone against the plain implementation; run orders that name a
layer twice or share a cache; a window group; and a toy mixer with state of its
own that is registered, built and stepped without touching the framework."""
import math
from dataclasses import dataclass, replace

import pytest
import torch

import harness
import tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _ctx(dtype):
    from prelude_b200.parts.registry import RunContext
    return RunContext(DEV, dtype)


def _store(tensors):
    from prelude_b200.weights.loader import WeightStore
    return WeightStore.from_tensors(tensors)


def _tol(dtype, ref):
    return 1e-5 * max(1.0, float(ref.abs().max())) if dtype == torch.float32 else 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_norm_part(dtype):
    from prelude_b200.config.spec import NormSpec
    from prelude_b200.parts.registry import make_part
    w = {"n.weight": 1 + 0.3 * torch.randn(200)}
    part = make_part("norm", NormSpec(200, 1e-4), "n")
    assert list(part.tensors()) == ["n.weight"]
    part.load(_store(w).get, _ctx(dtype))
    x = torch.randn(9, 200)
    want = plain.rms_norm(x, w["n.weight"], 1e-4)
    got = part.forward(x.to(DEV, dtype)).float().cpu()
    assert (got - plain.rms_norm(x.to(dtype).float(), w["n.weight"], 1e-4)).abs().max() <= _tol(dtype, want)
    res = torch.randn(9, 200, device=DEV)
    before = res.clone()
    y = part.add_forward(x.to(DEV, dtype), res)
    assert torch.allclose(res, before + x.to(DEV, dtype).float(), atol=1e-6) and y.dtype == dtype


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_feed_forward_part(dtype):
    from prelude_b200.config.spec import GatedMlpSpec
    from prelude_b200.parts.registry import make_part
    H, I = 72, 200
    w = {f"m.{n}.weight": (torch.randn(s) * 0.2).to(dtype) for n, s in
         (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I)))}
    part = make_part("feed_forward", GatedMlpSpec(H, I), "m")
    part.load(_store(w).get, _ctx(dtype))
    x = torch.randn(11, H).to(dtype)
    want = plain.swiglu_mlp(x.float(), {k: v.float() for k, v in w.items()}, "m")
    got = part.forward(x.to(DEV))
    if not isinstance(got, torch.Tensor):       # partial sums of a product whose K was cut into parts
        got = got.materialize(dtype)
    got = got.float().cpu()
    assert (got - want).abs().max() <= _tol(dtype, want)
    with pytest.raises(ValueError, match="activation"):
        make_part("feed_forward", GatedMlpSpec(H, I, activation="relu"), "m")


def _one_layer_setup(which, dtype, window=None):
    """Model spec, weights and a runner for a model cut down to its first layer."""
    from prelude_b200.config import load_model_config
    cfg, init, page = tiny.PARAMS[which]
    cfg = dict(cfg, num_hidden_layers=1)
    from prelude_b200.weights.random_init import random_tensors
    w = {k: v.to(dtype) for k, v in random_tensors(cfg, **init).items()}
    spec = load_model_config(cfg).to_model_spec()
    if window:
        blk = spec.blocks[0]
        spec = replace(spec, blocks=(replace(blk, mixer=replace(blk.mixer, window=window)),))
    return cfg, w, spec, page


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_attention_part_alone(which, dtype):
    """The mixer by itself: portions through the part against whole-sequence plain attention."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.parts.registry import make_part
    cfg, w, spec, page = _one_layer_setup(which, dtype)
    attn = make_part("mixer", spec.blocks[0].mixer, "model.layers.0.self_attn")
    assert set(attn.tensors()) <= set(w)
    attn.load(_store(w).get, _ctx(dtype))
    L = 45
    x = (torch.randn(L, cfg["hidden_size"]) * 0.5).to(dtype)
    cos, sin = plain.rope_tables(cfg["head_dim"], L, cfg["rope_theta"])
    want, _ = plain.attention_block(x.float(), {k: v.float() for k, v in w.items()}, "model.layers.0.self_attn", cfg, cos, sin)
    cache = CacheManager([attn.cache_need()], page, 16, 2, DEV, dtype)
    cache.add_request("r")
    got, start = [], 0
    for n in (7, 2, 16, 1, 19):
        cache.grow("r", start + n)
        batch = build_step_batch([StepItem("r", [0] * n, start)], cache.block_tables(["r"]), [cache.slot_of("r")], DEV, 10, 1000)
        got.append(attn.forward(x[start:start + n].to(DEV), batch, cache.layer_cache(0), True).float().cpu())
        start += n
    got = torch.cat(got)
    assert (got - want).abs().max() <= _tol(dtype, want)


def _run_model(spec, w, dtype, reqs, page, cuts=(harness.whole, harness.portions, harness.mixed)):
    from prelude_b200.engine.loading import build_model, make_runner
    model = build_model(spec, _store(w), dtype, DEV)
    outs = []
    for cut in cuts:
        schedule = cut(reqs)
        runner = make_runner(model, page_size=page, num_pages=harness.peak_tokens(schedule, page) // page, max_slots=8)
        outs.append(harness.run_schedule(runner, schedule))
        runner.cache.check()
        assert runner.cache.used_pages() == 0
    return outs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_run_order_may_name_a_layer_twice_and_share_a_cache(dtype):
    from prelude_b200.config import load_model_config
    from prelude_b200.config.spec import LayerCall
    from prelude_b200.weights.random_init import random_tensors
    cfg, init, page = tiny.PARAMS["B"]
    w = {k: v.to(dtype) for k, v in random_tensors(cfg, **init).items()}
    spec = load_model_config(cfg).to_model_spec()
    # layer 0, layer 1, layer 0 again (own cache), layer 2 reading the keys and values of the first call
    spec = replace(spec, order=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(2, cache=0, writes_cache=False)))
    order = [(0, None), (1, None), (0, None), (2, 0)]
    reqs = {"x": tiny.random_ids(37, cfg["vocab_size"], 1), "y": tiny.random_ids(50, cfg["vocab_size"], 2)}
    wf = {k: v.float() for k, v in w.items()}
    ref = {rid: plain.forward_logits(cfg, wf, toks, order=order) for rid, toks in reqs.items()}
    for got in _run_model(spec, w, dtype, reqs, page):
        for (rid, pos), row in got.items():
            want = ref[rid][pos]
            assert (row - want).abs().max() <= (1e-4 if dtype == torch.float32 else 3e-2 * float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_layers_with_a_window_have_pages_of_their_own_and_give_them_back(dtype):
    from prelude_b200.config import load_model_config
    from prelude_b200.weights.random_init import random_tensors
    cfg, init, page = tiny.PARAMS["A"]
    w = {k: v.to(dtype) for k, v in random_tensors(cfg, seed=5, std=0.08, norm_jitter=0.3).items()}
    spec = load_model_config(cfg).to_model_spec()
    window = 9
    b0, b1 = spec.blocks
    spec = replace(spec, blocks=(b0, replace(b1, mixer=replace(b1.mixer, window=window))))     # layer 1 sees 9 keys
    reqs = {"x": tiny.random_ids(60, cfg["vocab_size"], 3), "y": tiny.random_ids(41, cfg["vocab_size"], 4)}
    wf = {k: v.float() for k, v in w.items()}
    ref = {rid: plain.forward_logits(cfg, wf, toks, windows={1: window}) for rid, toks in reqs.items()}
    full = {rid: plain.forward_logits(cfg, wf, toks) for rid, toks in reqs.items()}
    assert (ref["x"][-1] - full["x"][-1]).abs().max() > 1e-3          # the window matters for these weights
    for got in _run_model(spec, w, dtype, reqs, page):
        for (rid, pos), row in got.items():
            want = ref[rid][pos]
            assert (row - want).abs().max() <= (1e-4 if dtype == torch.float32 else 3e-2 * float(want.abs().max()))
    # the window group really frees what has passed
    from prelude_b200.engine.loading import build_model, make_runner
    from prelude_b200.engine.runner import StepEntry
    runner = make_runner(build_model(spec, _store(w), dtype, DEV), page_size=page, num_pages=16, max_slots=2)
    assert len(runner.cache.groups) == 2
    runner.step([StepEntry("x", reqs["x"][:40], [])])
    held = {g.need.window: g.allocator.num_used for g in runner.cache.groups}
    assert held[None] == 10 and held[window] == 2                      # 40 tokens: 10 pages of 4; the next query reads keys from 32 on: 2 pages
    runner.finish("x")


# ---------------------------------------------------------------------------------------
# a toy mixer with state of its own, defined here, registered through the public hooks
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    kind: str = "toy_decay"


def _register_toy():
    from prelude_b200.parts.registry import StateNeed, register_part
    from prelude_b200.weights.loader import TensorReq

    @register_part("mixer", "toy_decay")
    class DecayMixer:
        """s_t = decay * s_{t-1} + W x_t ; y_t = s_t.  One state vector per request."""

        def __init__(self, spec, prefix):
            self.spec, self.prefix = spec, prefix

        def tensors(self):
            return {f"{self.prefix}.mix.weight": TensorReq((self.spec.hidden_size, self.spec.hidden_size))}

        def load(self, get, ctx):
            self.w = get(f"{self.prefix}.mix.weight").to(ctx.device, torch.float32)
            self.dtype = ctx.dtype

        def cache_need(self):
            return StateNeed((self.spec.hidden_size,), torch.float32)

        def forward(self, x, batch, cache, write_cache=True):
            assert cache.kind == "state"
            u = x.float() @ self.w.T
            out = torch.empty_like(u)
            row = 0
            for n, slot in zip(batch.q_lens.tolist(), batch.state_slots_host.tolist()):
                s = cache.state[slot]
                for t in range(row, row + n):
                    s = self.spec.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
                row += n
            return out.to(self.dtype)
    return DecayMixer


def _plain_toy(cfg, w, ids, decay):
    """Layer 0: Qwen3 attention block; layer 1: the decay mixer in place of attention."""
    wf = {k: v.float() for k, v in w.items()}
    L = len(ids)
    cos, sin = plain.rope_tables(cfg["head_dim"], L, cfg["rope_theta"])
    res = plain.embedding(torch.tensor(ids), wf["model.embed_tokens.weight"])
    res, _ = plain.decoder_block(res, wf, 0, cfg, cos, sin)
    x = plain.rms_norm(res, wf["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    u = x @ wf["model.layers.1.self_attn.mix.weight"].T
    s, ys = torch.zeros(cfg["hidden_size"]), []
    for t in range(L):
        s = decay * s + u[t]
        ys.append(s)
    res = res + torch.stack(ys)
    res = res + plain.swiglu_mlp(plain.rms_norm(res, wf["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"]), wf, "model.layers.1.mlp")
    return plain.rms_norm(res, wf["model.norm.weight"], cfg["rms_norm_eps"]) @ wf["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps():
    from prelude_b200.config import load_model_config
    from prelude_b200.parts.registry import unregister_part
    from prelude_b200.weights.random_init import random_tensors
    _register_toy()
    try:
        cfg, init, page = tiny.PARAMS["A"]
        spec = load_model_config(cfg).to_model_spec()
        b0, b1 = spec.blocks
        spec = replace(spec, blocks=(b0, replace(b1, mixer=DecaySpec(cfg["hidden_size"], 0.9))))
        w = random_tensors(cfg, **init)
        w = {k: v for k, v in w.items() if not k.startswith("model.layers.1.self_attn.")}
        w["model.layers.1.self_attn.mix.weight"] = torch.randn(cfg["hidden_size"], cfg["hidden_size"]) * 0.1
        reqs = {"x": tiny.random_ids(23, cfg["vocab_size"], 8), "y": tiny.random_ids(31, cfg["vocab_size"], 9),
                "z": tiny.random_ids(5, cfg["vocab_size"], 10)}
        ref = {rid: _plain_toy(cfg, w, toks, 0.9) for rid, toks in reqs.items()}
        # the weight check knows the toy's tensor and misses it when absent
        from prelude_b200.engine.loading import build_model
        from prelude_b200.weights.loader import WeightError
        with pytest.raises(WeightError, match="mix.weight"):
            build_model(spec, _store({k: v for k, v in w.items() if "mix" not in k}), torch.float32, DEV)
        for got in _run_model(spec, w, torch.float32, reqs, page):
            assert len(got) == 59
            for (rid, pos), row in got.items():
                assert (row - ref[rid][pos]).abs().max() <= 1e-4
        # slots are reused by later requests and start from zero again: run the mixed cut twice on one runner
        from prelude_b200.engine.loading import make_runner
        runner = make_runner(build_model(spec, _store(w), torch.float32, DEV), page_size=page, num_pages=32, max_slots=2)
        for _ in range(2):
            got = harness.run_schedule(runner, harness.mixed(reqs, max_live=2))
            for (rid, pos), row in got.items():
                assert (row - ref[rid][pos]).abs().max() <= 1e-4
        assert [g.members for g in runner.cache.groups] == [[0]] and list(runner.cache.state_tensors) == [1]
    finally:
        unregister_part("mixer", "toy_decay")


# ---------------------------------------------------------------------------------------
# a toy feed-forward with routing, and another position encoding, both defined here
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    expert_size: int
    n_experts: int
    kind: str = "toy_routed"


@dataclass(frozen=True)
class LinearAngleSpec:
    """Rotation angles that grow linearly in the pair index (not geometrically), over half of the head."""
    head_dim: int
    rotary_dim: int
    slope: float
    max_positions: int
    kind: str = "toy_linear_angle"


def _register_toy_ff_and_position():
    from prelude_b200.ops.linear import linear
    from prelude_b200.parts.registry import register_part
    from prelude_b200.weights.loader import TensorReq

    @register_part("feed_forward", "toy_routed")
    class RoutedFeedForward:
        """Every token goes to the one expert its router logit (32-bit) is largest for:
        y = p_e * down_e(relu(up_e x)), p = softmax(router x)."""

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
            choice = probs.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.spec.n_experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(linear(x[rows].contiguous(), self.up[e]))
                    out[rows] = (linear(h, self.down[e]).float() * probs[rows, e:e + 1]).to(x.dtype)
            return out

    @register_part("position", "toy_linear_angle")
    class LinearAngle:
        def __init__(self, spec, prefix=""):
            self.spec = spec
            self.cos = self.sin = None

        def tensors(self):
            return {}

        def load(self, get, ctx):
            s = self.spec
            ang = _linear_angles(s.rotary_dim, s.max_positions, s.slope)
            self.cos, self.sin = ang.cos().contiguous().to(ctx.device), ang.sin().contiguous().to(ctx.device)

        @property
        def rotary_dim(self):
            return self.spec.rotary_dim


def _linear_angles(rotary_dim, n_positions, slope):
    j = torch.arange(rotary_dim // 2, dtype=torch.float32)
    return torch.arange(n_positions, dtype=torch.float32)[:, None] * (slope * (1.0 + j))[None, :]


def _plain_routed_and_linear_angle(cfg, w, ids, n_experts, rotary_dim, slope):
    """Layer 0: attention rotating the first ``rotary_dim`` elements of every head by linearly spaced angles,
    dense feed-forward; layer 1: the same attention, routed feed-forward.  Whole sequence, no cache."""
    wf = {k: v.float() for k, v in w.items()}
    L, eps = len(ids), cfg["rms_norm_eps"]
    nH, nKV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    ang = _linear_angles(rotary_dim, L, slope)
    cos, sin = ang.cos(), ang.sin()

    def rotate(x):                                           # [L, heads, D]: the first rotary_dim elements, half-split pairs
        return torch.cat([plain.apply_rope(x[..., :rotary_dim], cos, sin), x[..., rotary_dim:]], dim=-1)

    res = plain.embedding(torch.tensor(ids), wf["model.embed_tokens.weight"])
    for i in range(2):
        p = f"model.layers.{i}"
        x = plain.rms_norm(res, wf[f"{p}.input_layernorm.weight"], eps)
        q = plain.rms_norm((x @ wf[f"{p}.self_attn.q_proj.weight"].T).reshape(L, nH, D), wf[f"{p}.self_attn.q_norm.weight"], eps)
        k = plain.rms_norm((x @ wf[f"{p}.self_attn.k_proj.weight"].T).reshape(L, nKV, D), wf[f"{p}.self_attn.k_norm.weight"], eps)
        v = (x @ wf[f"{p}.self_attn.v_proj.weight"].T).reshape(L, nKV, D)
        o = plain.causal_attention(rotate(q), rotate(k), v, 1.0 / math.sqrt(D))
        res = res + o.reshape(L, nH * D) @ wf[f"{p}.self_attn.o_proj.weight"].T
        x = plain.rms_norm(res, wf[f"{p}.post_attention_layernorm.weight"], eps)
        if i == 0:
            res = res + plain.swiglu_mlp(x, wf, f"{p}.mlp")
        else:
            probs = torch.softmax(x @ wf[f"{p}.mlp.router.weight"].T, dim=-1)
            choice = probs.argmax(dim=-1)
            y = torch.zeros_like(x)
            for t in range(L):
                e = int(choice[t])
                h = torch.relu(x[t] @ wf[f"{p}.mlp.experts.{e}.up.weight"].T)
                y[t] = probs[t, e] * (h @ wf[f"{p}.mlp.experts.{e}.down.weight"].T)
            res = res + y
    return plain.rms_norm(res, wf["model.norm.weight"], eps) @ wf["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_toy_routed_feed_forward_and_another_position_encoding(dtype):
    """Two more parts from outside the package: a feed-forward that routes every token to one of three experts,
    and a position encoding with its own angles over half of the head.  They are registered through the public
    hook, chosen by the specs of single layers, and the model steps through every way of cutting."""
    from prelude_b200.config import load_model_config
    from prelude_b200.parts.registry import unregister_part
    from prelude_b200.weights.random_init import random_tensors
    _register_toy_ff_and_position()
    try:
        cfg, init, page = tiny.PARAMS["A"]
        H, D, E, I = cfg["hidden_size"], cfg["head_dim"], 3, 40
        spec = load_model_config(cfg).to_model_spec()
        pos = LinearAngleSpec(D, D // 2, 0.07, cfg["max_position_embeddings"])
        b0, b1 = spec.blocks
        b0 = replace(b0, mixer=replace(b0.mixer, position=pos))
        b1 = replace(b1, mixer=replace(b1.mixer, position=pos), feed_forward=RoutedSpec(H, I, E))
        spec = replace(spec, blocks=(b0, b1))
        g = torch.Generator().manual_seed(5)
        w = {k: v for k, v in random_tensors(cfg, **init).items() if not k.startswith("model.layers.1.mlp.")}
        w["model.layers.1.mlp.router.weight"] = torch.randn(E, H, generator=g)
        for e in range(E):
            w[f"model.layers.1.mlp.experts.{e}.up.weight"] = torch.randn(I, H, generator=g) * 0.1
            w[f"model.layers.1.mlp.experts.{e}.down.weight"] = torch.randn(H, I, generator=g) * 0.1
        w = {k: v.to(dtype) for k, v in w.items()}
        reqs = {"x": tiny.random_ids(29, cfg["vocab_size"], 21), "y": tiny.random_ids(18, cfg["vocab_size"], 22)}
        ref = {rid: _plain_routed_and_linear_angle(cfg, w, toks, E, D // 2, 0.07) for rid, toks in reqs.items()}
        # the other position encoding matters: the model's own rotary tables give other logits
        assert (ref["x"][-1] - plain.forward_logits(cfg, {k: v.float() for k, v in random_tensors(cfg, **init).items()}, reqs["x"])[-1]).abs().max() > 1e-3
        for got in _run_model(spec, w, dtype, reqs, page):
            assert len(got) == 47
            for (rid, p), row in got.items():
                want = ref[rid][p]
                assert (row - want).abs().max() <= (2e-4 if dtype == torch.float32 else 4e-2 * float(want.abs().max()))
    finally:
        unregister_part("feed_forward", "toy_routed")
        unregister_part("position", "toy_linear_angle")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_position_encoding_that_turns_adjacent_pairs(dtype):
    """A position part from outside the package whose angle j turns elements 2 j and 2 j + 1 (not j and j + half):
    it says so with ``interleaved = True`` and the attention mixer's kernel pairs accordingly.  Against a plain
    whole-sequence computation written here, through every way of cutting."""
    from prelude_b200.config import load_model_config
    from prelude_b200.parts.registry import register_part, unregister_part
    from prelude_b200.weights.random_init import random_tensors

    @dataclass(frozen=True)
    class AdjacentSpec:
        head_dim: int
        theta: float
        max_positions: int
        kind: str = "toy_adjacent_pairs"

    def angles(D, n, theta):
        inv = torch.tensor([1.0 / theta ** (i / D) for i in range(0, D, 2)], dtype=torch.float64).float()
        return torch.arange(n, dtype=torch.float32)[:, None] * inv[None]

    @register_part("position", "toy_adjacent_pairs")
    class AdjacentPairs:
        interleaved = True

        def __init__(self, spec, prefix=""):
            self.spec = spec
            self.cos = self.sin = None

        def tensors(self):
            return {}

        def load(self, get, ctx):
            ang = angles(self.spec.head_dim, self.spec.max_positions, self.spec.theta)
            self.cos, self.sin = ang.cos().contiguous().to(ctx.device), ang.sin().contiguous().to(ctx.device)

        @property
        def rotary_dim(self):
            return self.spec.head_dim

    try:
        cfg, init, page = tiny.PARAMS["B"]
        D, nH, nKV, eps = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
        spec = load_model_config(cfg).to_model_spec()
        pos = AdjacentSpec(D, 5000.0, cfg["max_position_embeddings"])
        spec = replace(spec, blocks=tuple(replace(b, mixer=replace(b.mixer, position=pos)) for b in spec.blocks))
        w = {k: v.to(dtype) for k, v in random_tensors(cfg, **init).items()}
        wf = {k: v.float() for k, v in w.items()}

        def plain_logits(ids):
            L = len(ids)
            ang = angles(D, L, 5000.0)
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def turn(x):                                                    # [L, heads, D], pairs (2j, 2j + 1)
                a, b = x[..., 0::2], x[..., 1::2]
                return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).reshape(x.shape)

            res = plain.embedding(torch.tensor(ids), wf["model.embed_tokens.weight"])
            for i in range(cfg["num_hidden_layers"]):
                p = f"model.layers.{i}"
                x = plain.rms_norm(res, wf[f"{p}.input_layernorm.weight"], eps)
                q = plain.rms_norm((x @ wf[f"{p}.self_attn.q_proj.weight"].T).reshape(L, nH, D), wf[f"{p}.self_attn.q_norm.weight"], eps)
                k = plain.rms_norm((x @ wf[f"{p}.self_attn.k_proj.weight"].T).reshape(L, nKV, D), wf[f"{p}.self_attn.k_norm.weight"], eps)
                v = (x @ wf[f"{p}.self_attn.v_proj.weight"].T).reshape(L, nKV, D)
                o = plain.causal_attention(turn(q), turn(k), v, 1.0 / math.sqrt(D))
                res = res + o.reshape(L, nH * D) @ wf[f"{p}.self_attn.o_proj.weight"].T
                res = res + plain.swiglu_mlp(plain.rms_norm(res, wf[f"{p}.post_attention_layernorm.weight"], eps), wf, f"{p}.mlp")
            return plain.rms_norm(res, wf["model.norm.weight"], eps) @ wf["lm_head.weight"].T

        reqs = {"x": tiny.random_ids(41, cfg["vocab_size"], 61), "y": tiny.random_ids(19, cfg["vocab_size"], 62)}
        ref = {rid: plain_logits(toks) for rid, toks in reqs.items()}
        half_split = plain.forward_logits(dict(cfg, rope_theta=5000.0), wf, reqs["x"])
        assert (ref["x"][-1] - half_split[-1]).abs().max() > 1e-3          # the pairing matters
        for got in _run_model(spec, w, dtype, reqs, page):
            for (rid, p), row in got.items():
                want = ref[rid][p]
                assert (row - want).abs().max() <= (2e-4 if dtype == torch.float32 else 4e-2 * float(want.abs().max()))
    finally:
        unregister_part("position", "toy_adjacent_pairs")
