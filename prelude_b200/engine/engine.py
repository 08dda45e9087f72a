"""The Python entry point: ``Engine(model_dir).generate(prompts, ...)``.

The reference has no Python binding; the shape follows its engine interface
(``InferenceEngine::generate``, crates/prelude-core/src/engine/mod.rs:76-132)
and its request and result records (crates/prelude-core/src/types.rs:400-434):
a request is token ids plus sampling options, a result is the generated ids, a
finish reason, token counts and timings.  Option names and defaults are those
of the reference's command line (crates/prelude-server/src/main.rs:15-183).

``generate`` runs the reference's loop (crates/prelude-core/src/engine/run/ar.rs:205-387):
schedule a step, build the batch, run it, sample where a request reached its
last token, apply the stop checks, free what finished.  Tokenisation lies
outside: prompts are token ids.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_model_config
from ..ops.library import require_device
from ..sampling.sampler import Sampler, sampling_mode
from .graph import DecodeGraphs
from .loading import load_model, parse_dtype
from ..parts.model import DecoderModel
from .batch import raise_on_status
from .runner import ModelRunner, StepEntry
from .scheduler import ScheduledItem, CachePoolView, SamplingParams, Scheduler, SchedulerConfig


@dataclass
class GenerateResult:
    request_id: object
    token_ids: List[int]
    finish_reason: str                  # "eos" | "stop" | "length" | "abort" | "cache_full"
    prompt_tokens: int
    completion_tokens: int
    ttft_ms: float = 0.0                # first token after the request was handed in
    total_ms: float = 0.0
    preemptions: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    decode_steps: int = 0
    graph_steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    pages_total: int = 0
    pages_in_use_peak: int = 0
    step_ms_total: float = 0.0
    h2d_bytes: int = 0                  # bytes copied host to device for the steps' inputs (counted from the tensors copied)
    d2h_bytes: int = 0                  # bytes read back: sampled tokens and the status word


def _activation_reserve_bytes(model: DecoderModel, max_tokens: int, max_rows: int) -> int:
    """A generous bound on what one step allocates beside weights and cache.  A mixer or feed-forward says what it
    allocates per token (``activation_bytes_per_token(element size)``); one that does not say is taken to use
    sixteen rows of the hidden width in 32-bit, so that an unknown part never counts as nothing."""
    spec = model.spec
    elem = 2 if model.ctx.dtype == torch.bfloat16 else 4
    widest = 0
    for b in model.blocks:
        per_token = 4 * spec.hidden_size * 4              # residual, two normed copies, a delta
        inner = b.parts() if callable(getattr(b, "parts", None)) else ()
        for part in inner:
            say = getattr(part, "activation_bytes_per_token", None)
            if callable(say):
                per_token += int(say(elem))
            elif callable(getattr(part, "forward", None)) and not hasattr(part, "add_forward"):
                per_token += 16 * spec.hidden_size * 4
        widest = max(widest, per_token)
    return max_tokens * widest + 3 * max_rows * spec.vocab_size * 4 + (1 << 30)


class Engine:
    def __init__(self, model: str, dtype: str = "bf16", device: str = "cuda:0", page_size: int = 16,
                 num_pages: Optional[int] = None, gpu_memory_utilization: float = 0.9,
                 max_running_requests: int = 256, max_num_batched_tokens: int = 8192,
                 long_prefill_token_threshold: int = 0, max_total_tokens: int = 0, decode_reservation_cap: int = 0,
                 decode_priority_max_remaining_tokens: int = 4, cuda_graph: bool = True, cuda_graph_max_bs: int = 64,
                 max_model_len: Optional[int] = None, decode_burst: int = 8, random_weights_seed: Optional[int] = None):
        """``model`` is a folder with config.json and safetensors files (or a
        DecoderModel that is already on the device).  With ``random_weights_seed`` the folder's
        config.json alone is read and the weights are drawn from that seed on the device.

        ``num_pages`` fixes the cache size; without it the cache takes what
        ``gpu_memory_utilization`` of the device leaves after the weights and a
        reserve for one step's activations
        (crates/prelude-core/src/scheduler/components/cache/manager.rs:240-280).
        ``max_model_len`` caps a request's length below max_position_embeddings.
        """
        require_device()
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        if isinstance(model, DecoderModel):
            # an already built model (random weights made on the device, toy architectures in tests)
            self.config = None
            self.model = model
            self.device, self.dtype = model.ctx.device, model.ctx.dtype
        else:
            self.config = load_model_config(model)
            self.model = load_model(model, self.dtype, self.device, random_weights_seed=random_weights_seed)
        spec = self.model.spec
        self.max_model_len = min(max_model_len or spec.max_positions, spec.max_positions)
        needs = self.model.cache_needs()
        elem = 2 if self.dtype == torch.bfloat16 else 4
        if num_pages is None:
            per_page = max(1, CacheManager.bytes_per_page(needs, page_size, elem))
            free, total = torch.cuda.mem_get_info(self.device)
            budget = free - int((1.0 - gpu_memory_utilization) * total) \
                - _activation_reserve_bytes(self.model, max_num_batched_tokens, max_running_requests)
            num_pages = max(16, budget // per_page)
            # no more than every request slot at full length could use
            num_pages = min(num_pages, max_running_requests * -(-self.max_model_len // page_size))
        # what the parts allow: a model with a part that cannot be recorded has its steps launched kernel by kernel
        self.caps = self.model.runtime_caps()
        cuda_graph = bool(cuda_graph and self.caps.cuda_graph)
        self.cache = CacheManager(needs, page_size, int(num_pages), max_running_requests, self.device, self.dtype,
                                  max_request_tokens=self.max_model_len if cuda_graph else None)
        self.runner = ModelRunner(self.model, self.cache)
        self.sched_config = SchedulerConfig(
            max_running_requests=max_running_requests, max_num_batched_tokens=max_num_batched_tokens,
            long_prefill_token_threshold=long_prefill_token_threshold, max_total_tokens=max_total_tokens,
            decode_reservation_cap=decode_reservation_cap or self.max_model_len,
            decode_priority_max_remaining_tokens=decode_priority_max_remaining_tokens, page_size=page_size)
        self.sampler = Sampler(self.device)
        self.eos_token_ids = tuple(spec.eos_token_ids)
        self.cuda_graph = cuda_graph
        self.graphs = DecodeGraphs(self.runner, cuda_graph_max_bs) if cuda_graph else None
        if cuda_graph:
            self.runner.enable_step_graphs()
        # Runs of decode steps queued without the host in between (see _burst_length): up to this many
        self.decode_burst = max(1, int(decode_burst))
        self.burst_graphs = (DecodeGraphs(self.runner, cuda_graph_max_bs, self_feeding=True)
                             if cuda_graph and self.decode_burst > 1 else None)
        self._stats = EngineStats(pages_total=int(num_pages))
        self._next_id = 0
        # one scheduler for the engine's life: requests arrive and leave while others run
        self.sched = Scheduler(self.sched_config, CachePoolView(self.cache))
        self._inbox: deque = deque()                 # (id, prompt, params, time handed in), from any thread
        self._aborts: deque = deque()
        self._inbox_lock = threading.Lock()
        self._submitted_at: Dict[int, float] = {}
        self._first_token_at: Dict[int, float] = {}
        self._done: Dict[int, GenerateResult] = {}   # finished requests that nobody has taken yet

    # -- the raw step function, for tests and tools ---------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        return self.runner.step(entries)

    def finish(self, request_id) -> None:
        self.runner.finish(request_id)

    def stats(self) -> EngineStats:
        return self._stats

    def warmup(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """Capture the decode step for the given batch sizes (default: every size up to
        ``max_running_requests`` and ``cuda_graph_max_bs``) before the first request needs
        them: a capture takes a few hundred milliseconds, which a request would otherwise
        wait for the first time its batch size comes up.  Runs short dummy generations;
        returns the sizes captured.  (The reference warms its graphs up at start-up as well,
        crates/prelude-cuda/src/cuda_graph.rs:84-112, one capture per batch size up to cuda_graph_max_bs.)"""
        if self.graphs is None:
            return []
        limit = min(self.graphs.max_bs, self.sched_config.max_running_requests)
        sizes = sorted({int(b) for b in (batch_sizes if batch_sizes is not None else range(1, limit + 1))
                        if 1 <= int(b) <= limit})
        done = []
        for bs in sizes:
            if bs in self.graphs.graphs and self.graphs.graphs[bs].graph is not None:
                continue
            # two tokens: the second comes from a single captured step; five: from a queued run of steps
            self.generate([[0]] * bs, temperature=0.0, max_new_tokens=2, ignore_eos=True)
            if self.burst_graphs is not None:
                self.generate([[0]] * bs, temperature=0.0, max_new_tokens=5, ignore_eos=True)
            if bs in self.graphs.graphs:
                done.append(bs)
        return done

    def warmup_prompt_steps(self, token_counts: Optional[Sequence[int]] = None) -> List[int]:
        """Capture the pieces of prompt steps for the buckets of the given token counts (default: every bucket up
        to the limit) before a request needs them: the first step of a bucket records its pieces, which takes
        tens of milliseconds.  Runs one dummy prompt per bucket; returns the buckets captured."""
        from .step_graph import bucket_of
        sg = self.runner.step_graphs
        if sg is None:
            return []
        if token_counts is None:
            token_counts, n = [], 1
            while bucket_of(n) <= sg.max_tokens:
                token_counts.append(bucket_of(n))
                n = bucket_of(n) + 1
        done = []
        for n in sorted({bucket_of(int(t)) for t in token_counts}):
            room = min(self.max_model_len - 2, self.cache.num_pages * self.cache.page_size - 2,
                       self.sched_config.max_num_batched_tokens)
            if n < 2 or n > sg.max_tokens or n > room or (n in sg.graphs and sg.graphs[n].captured):
                continue
            self.generate([[0] * n], temperature=0.0, max_new_tokens=1, ignore_eos=True)
            if n in sg.graphs and sg.graphs[n].captured:
                done.append(n)
        return done

    # -- requests that come and go while the engine runs -------------------------------------
    def submit(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None, **options) -> int:
        """Hand in one request (token ids, sampling options as in ``generate``); returns its id.  The request
        joins the batch at the next ``step_once``, beside whatever is running, as in the reference's loop
        (crates/prelude-core/src/engine/run/ar.rs:205-387 drains new requests every iteration; admission
        :501-558).  May be called from another thread than the one that steps the engine; a run of queued
        decode steps in flight is cut short so that the newcomer does not wait for all of it."""
        params = self._params(sampling, options)
        prompt = list(prompt)
        vocab = self.model.spec.vocab_size
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if any((not isinstance(t, int)) or t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"prompt token ids must be integers in [0, {vocab})")
        if len(prompt) >= self.max_model_len:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room below the length limit {self.max_model_len}")
        with self._inbox_lock:
            rid = self._next_id
            self._next_id += 1
            self._inbox.append((rid, prompt, params, time.perf_counter()))
        return rid

    def abort(self, request_id: int) -> None:
        """End a request wherever it is - waiting, in the middle of its prompt, decoding: at the next
        ``step_once`` its pages and slot go back and its result carries the reason "abort"
        (ar.rs:436-444).  Unknown and finished ids are ignored.  May be called from another thread."""
        with self._inbox_lock:
            self._aborts.append(request_id)

    def has_work(self) -> bool:
        return bool(self._inbox or self._aborts or self.sched.has_work())

    def _mail_waiting(self) -> bool:
        return bool(self._inbox or self._aborts)

    def _drain_mail(self) -> None:
        with self._inbox_lock:
            arrivals, self._inbox = list(self._inbox), deque()
            aborts, self._aborts = list(self._aborts), deque()
        for rid, prompt, params, t_in in arrivals:
            self.sched.add_request(rid, prompt, params, self.max_model_len)
            self._submitted_at[rid] = t_in
        for rid in aborts:
            self.sched.abort(rid)

    def step_once(self) -> List[GenerateResult]:
        """One iteration of the loop: take in what was submitted or aborted, schedule a step, run it (or a run of
        queued decode steps), sample, apply the stop checks, free what finished.  Returns the results of the
        requests that ended in it."""
        self._drain_mail()
        sched = self.sched
        finished: List[GenerateResult] = []
        if not sched.has_work():
            self._collect(finished)
            return finished
        try:
            items = sched.schedule()
            self._collect(finished)
            if not items:
                if sched.has_work():
                    raise RuntimeError("the scheduler has work but could schedule nothing")
                return finished
            burst = self._burst_length(sched, items)
            if burst >= 2:
                for j, tokens in enumerate(self._run_burst(items, burst)):
                    for it, tok in zip(items, tokens):
                        sched.on_step_done(it if j == 0 else ScheduledItem(it.seq, 1, it.start + j), tok, self.eos_token_ids)
            else:
                tokens = self._run_step(items)
                now = time.perf_counter()
                for it, tok in zip(items, tokens):
                    if tok is not None:
                        self._first_token_at.setdefault(it.seq.request_id, now)
                    sched.on_step_done(it, tok, self.eos_token_ids)
        except BaseException:
            # a step failed (a kernel's status word, an interrupt, ...): what the requests hold goes back, so that
            # the engine can be used again; their results say "abort"
            for seq in list(sched.running) + list(sched.waiting):
                sched.abort(seq.request_id)
            self._collect(finished)
            for r in finished:
                self._done[r.request_id] = r
            raise
        self._collect(finished)
        self._stats.preemptions = sched.stats["preemptions"]
        return finished

    def run_until_idle(self) -> List[GenerateResult]:
        """Step until nothing is waiting or running; the results in the order the requests ended."""
        out: List[GenerateResult] = []
        while self.has_work():
            out.extend(self.step_once())
        return out

    def result(self, request_id: int) -> Optional[GenerateResult]:
        """The result of a finished request that no ``step_once`` caller has taken (``generate`` keeps the results
        of requests that are not its own here); None while it runs."""
        return self._done.pop(request_id, None)

    # -- generation ---------------------------------------------------------------------
    def _params(self, sampling: Optional[SamplingParams], options: Dict[str, object]) -> SamplingParams:
        q = SamplingParams(**vars(sampling or SamplingParams()))
        for k in ("max_new_tokens", "temperature", "top_p", "top_k", "seed", "ignore_eos"):
            if options.get(k) is not None:
                setattr(q, k, options[k])
        if options.get("stop_token_ids") is not None:
            q.stop_token_ids = tuple(options["stop_token_ids"])
        unknown = set(options) - {"max_new_tokens", "temperature", "top_p", "top_k", "seed", "ignore_eos", "stop_token_ids"}
        if unknown:
            raise TypeError(f"unknown sampling options {sorted(unknown)}")
        return q

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling: Union[None, SamplingParams, Sequence[SamplingParams]] = None, *,
                 max_new_tokens: Optional[int] = None, temperature: Optional[float] = None,
                 top_p: Optional[float] = None, top_k: Optional[int] = None, seed: Optional[int] = None,
                 stop_token_ids: Optional[Sequence[int]] = None, ignore_eos: Optional[bool] = None
                 ) -> Union[GenerateResult, List[GenerateResult]]:
        """Generate for one prompt (a list of token ids) or several (a list of
        lists).  ``sampling`` gives the options per request or for all; keyword
        options override it.  Built on ``submit`` and ``step_once``: requests that
        others submit meanwhile run in the same batches."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if isinstance(sampling, SamplingParams) or sampling is None:
            plist_params = [sampling] * len(plist)
        else:
            plist_params = list(sampling)
            if len(plist_params) != len(plist):
                raise ValueError("one SamplingParams per prompt")
        options = dict(max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p, top_k=top_k, seed=seed,
                       stop_token_ids=stop_token_ids, ignore_eos=ignore_eos)
        checked = [(p, self._params(sp, options)) for p, sp in zip(plist, plist_params)]
        vocab = self.model.spec.vocab_size
        for prompt, _ in checked:                           # all of them before any is handed in
            if any((not isinstance(t, int)) or t < 0 or t >= vocab for t in prompt):
                raise ValueError(f"prompt token ids must be integers in [0, {vocab})")
        ids = [self.submit(prompt, q) for prompt, q in checked]
        mine: Dict[int, GenerateResult] = {}
        try:
            while len(mine) < len(ids):
                if not self.has_work():
                    raise RuntimeError("requests are unfinished and the engine has no work")
                for r in self.step_once():
                    if r.request_id in ids:
                        mine[r.request_id] = r
                    else:
                        self._done[r.request_id] = r
        except BaseException:
            for rid in ids:
                self._done.pop(rid, None)
            raise
        results = [mine[r] for r in ids]
        return results[0] if single else results

    def _collect(self, into: List[GenerateResult]) -> None:
        now = time.perf_counter()
        for seq in self.sched.drain_finished():
            rid = seq.request_id
            t0 = self._submitted_at.pop(rid, now)
            first = self._first_token_at.pop(rid, now)
            into.append(GenerateResult(
                rid, list(seq.output), seq.finish_reason or "abort", len(seq.prompt), len(seq.output),
                ttft_ms=(first - t0) * 1e3, total_ms=(now - t0) * 1e3, preemptions=seq.preempt_count))

    def _burst_length(self, sched: Scheduler, items) -> int:
        """How many decode steps may be queued on the device without the host looking at the
        tokens in between.  A graph launch costs the host about as much as a tenth of a step
        of a 4B model; with the sampled token fed to the next step on the device, the launches
        of a run overlap the steps before them.  A run is taken when nothing could change the
        batch before it ends: every running request is in the step and decoding, nobody is
        waiting, sampling runs on the device (greedy or temperature), every request still has
        that many tokens to go (one that stops early - end of sequence, a stop token - has
        its later tokens dropped), and the pages for all of it are free."""
        if self.burst_graphs is None or sched.waiting or len(items) != len(sched.running) or self._mail_waiting():
            return 1
        if not all(it.n_tokens == 1 and it.samples for it in items):
            return 1
        if any(sampling_mode(it.seq.params.temperature, it.seq.params.top_k, it.seq.params.top_p) not in ("greedy", "all")
               for it in items):
            return 1
        k = min(self.decode_burst, min(it.seq.max_new_tokens - len(it.seq.output) for it in items))
        if k < 2 or not self.burst_graphs.usable(len(items), max(it.start + k for it in items)):
            return 1
        demand: Dict[int, int] = {}
        for it in items:
            rid = it.seq.request_id
            if not self.cache.has_request(rid):
                return 1
            for gid, n in self.cache.pages_needed(rid, it.start + k).items():
                demand[gid] = demand.get(gid, 0) + n
        if any(n > self.cache.groups[gid].allocator.num_free for gid, n in demand.items()):
            return 1
        return k

    def _run_burst(self, items, k: int) -> List[List[int]]:
        """``k`` decode steps of the same requests, queued at once; the tokens of every step."""
        t0 = time.perf_counter()
        entries = [StepEntry(it.seq.request_id, it.seq.tokens[it.start:it.start + 1], [0]) for it in items]
        starts = self.runner.reserve(entries)
        for it in items:
            self.cache.grow(it.seq.request_id, it.start + k)
        flushed = self.cache.flush_table_updates()
        self.cache.zero_fresh_state()
        g = self.burst_graphs.get(len(items))
        g.load([e.tokens[0] for e in entries], starts, [self.cache.slot_of(e.request_id) for e in entries],
               [it.seq.params.temperature for it in items], [it.seq.params.seed for it in items],
               [len(it.seq.output) for it in items])
        steps = g.replay_burst(k, stop=self._mail_waiting)
        if len(steps) < k:
            # the run was cut short (somebody arrived or was aborted): the cache holds what the steps that ran wrote
            k = len(steps)
            for it in items:
                self.cache.rewind(it.seq.request_id, it.start + k)
        now = time.perf_counter()
        for it in items:
            self._first_token_at.setdefault(it.seq.request_id, now)
        for e in entries:
            self.cache.trim(e.request_id)
        st = self._stats
        st.h2d_bytes += g.h2d_bytes + 8 * flushed          # one load for the whole run
        st.d2h_bytes += 4 * (k * len(items) + 1)
        st.graph_steps += k
        st.steps += k
        st.decode_steps += k
        st.generated_tokens += k * len(items)
        st.pages_in_use_peak = max(st.pages_in_use_peak, self.cache.used_pages())
        st.step_ms_total += (time.perf_counter() - t0) * 1e3
        return steps

    def _run_step(self, items) -> List[Optional[int]]:
        """Run one scheduled step; returns the sampled token per item (None
        where the portion did not reach the request's end)."""
        t0 = time.perf_counter()
        entries, rows = [], []
        for it in items:
            toks = it.seq.tokens[it.start:it.start + it.n_tokens]
            entries.append(StepEntry(it.seq.request_id, toks, [it.n_tokens - 1] if it.samples else []))
            if it.samples:
                rows.append(it)
        decode_only = all(it.n_tokens == 1 and it.samples for it in items)
        temps = [it.seq.params.temperature for it in rows]
        top_ks, top_ps = [it.seq.params.top_k for it in rows], [it.seq.params.top_p for it in rows]
        seeds, counters = [it.seq.params.seed for it in rows], [len(it.seq.output) for it in rows]
        st = self._stats
        if (decode_only and self.graphs is not None
                and self.graphs.usable(len(items), max(it.start + 1 for it in items))):
            # the captured step: same reservation, same kernels, fixed buffers
            starts = self.runner.reserve(entries)
            flushed = self.cache.flush_table_updates()
            self.cache.zero_fresh_state()
            g = self.graphs.get(len(items))
            st.h2d_bytes += g.h2d_bytes + 8 * flushed
            st.d2h_bytes += g.d2h_bytes
            g.load([e.tokens[0] for e in entries], starts, [self.cache.slot_of(e.request_id) for e in entries],
                   temps, seeds, counters)
            g.replay()
            sampled = g.fetch()
            if any(sampling_mode(t, k, p) in ("top_p", "top_k_top_p") for t, k, p in zip(temps, top_ks, top_ps)):
                sampled = self.sampler.sample(g.logits, temps, top_ks, top_ps, seeds, counters)
            for e in entries:
                self.cache.trim(e.request_id)
            st.graph_steps += 1
        else:
            logits = self.runner.step(entries, check_status=False)
            sampled = self.sampler.sample(logits, temps, top_ks, top_ps, seeds, counters) if rows else []
            raise_on_status(int(self.runner.last_batch.status.item()))
            st.h2d_bytes += self.runner.last_batch.h2d_bytes
            st.d2h_bytes += 4 * (len(rows) + 1)
        st.steps += 1
        st.decode_steps += 1 if decode_only else 0
        st.generated_tokens += len(rows)
        st.prompt_tokens += sum(it.n_tokens for it in items if it.seq.prefilling and it.start < len(it.seq.prompt))
        st.pages_in_use_peak = max(st.pages_in_use_peak, self.cache.used_pages())
        st.step_ms_total += (time.perf_counter() - t0) * 1e3
        out: List[Optional[int]] = []
        k = 0
        for it in items:
            if it.samples:
                out.append(int(sampled[k]))
                k += 1
            else:
                out.append(None)
        return out
