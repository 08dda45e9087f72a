"""Continuous batching: who runs in the next step, and with how many tokens.

Pure host logic; it never touches a tensor.  It follows the reference's chunked
scheduler (crates/prelude-core/src/scheduler/admission.rs:101-194, 297-428;
state.rs:85-117, 197-243; preemption.rs:7-116):

1. Running requests first: a request whose cache lags behind its tokens gets a
   portion ``min(pending, per-request cap, what is left of the step's token
   budget)``; a decoding request has exactly one pending token.
2. Then waiting requests, first come first served, while request slots, token
   budget and pages allow.  A request is admitted only if the pages of its
   whole prompt plus a capped reservation for what it will generate, plus the
   pages that already admitted prompts still have to take, fit the free pool.
   Nothing is admitted while every decoding request is within a few tokens of
   its end (short tails finish first).
3. If nothing at all could be scheduled and the waiting queue is not empty, a
   single token of its head is forced so that the system moves.

When pages run out:

* a waiting request simply waits (rule 2);
* a running request that cannot get the page its next tokens need sits the step
  out;
* if a step ends up empty because of that, one running request is preempted
  (never the oldest; the one preempted most often, then the newest): its pages
  go back, it returns to the head of the waiting queue with the tokens it has
  generated, and when it is admitted again it prefills prompt *and* generated
  tokens, so its cache is rebuilt in full.  (The reference re-prefills the
  prompt only and never rebuilds the keys of the generated tokens,
  state.rs:163-166 against engine/run/ar.rs:772-776.)
* a lone request that does not fit the pool even by itself is finished with the
  reason ``cache_full``.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple


@dataclass
class SamplingParams:
    """Per-request sampling options, with the reference's names and defaults
    (crates/prelude-core/src/scheduler/state.rs:6-32; seed: constants.rs:4)."""
    temperature: float = 0.7
    top_p: float = 1.0
    top_k: Optional[int] = None
    seed: int = 42
    max_new_tokens: int = 4096
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False


@dataclass
class SchedulerConfig:
    """The reference's knobs with its command-line defaults
    (crates/prelude-server/src/main.rs:40-122, 327-359)."""
    max_running_requests: int = 256
    max_num_batched_tokens: int = 8192
    long_prefill_token_threshold: int = 0        # per-request portion cap; 0: none
    max_total_tokens: int = 0                    # tokens held by running requests; 0: bounded by pages only
    decode_reservation_cap: int = 4096
    decode_priority_max_remaining_tokens: int = 4
    page_size: int = 16


WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Sequence:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    arrival: int = 0
    output: List[int] = field(default_factory=list)
    computed: int = 0                # tokens whose keys and values are in the cache
    status: str = WAITING
    finish_reason: Optional[str] = None
    preempt_count: int = 0
    scheduled: int = 0               # tokens given out by the last schedule() and not yet confirmed

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def pending(self) -> int:
        """Tokens that have not been through the model yet."""
        return self.total_len - self.computed

    @property
    def remaining_new(self) -> int:
        return max(0, self.max_new_tokens - len(self.output))

    @property
    def prefilling(self) -> bool:
        return self.pending > 1 or not self.output


@dataclass
class ScheduledItem:
    seq: Sequence
    n_tokens: int
    start: int

    @property
    def samples(self) -> bool:
        """True when the portion reaches the request's last token: its logits are wanted."""
        return self.start + self.n_tokens == self.seq.total_len


class PagePool:
    """What the scheduler needs to know about the cache.  ``CacheManager``
    satisfies it; tests may pass a plain counter."""

    def free_pages(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def pages_held(self, rid) -> int:  # pragma: no cover
        raise NotImplementedError

    def release(self, rid) -> None:  # pragma: no cover
        raise NotImplementedError


class CachePoolView(PagePool):
    """Adapter over a CacheManager: counts in pages of its tightest group."""

    def __init__(self, cache):
        self.cache = cache

    def free_pages(self) -> int:
        return self.cache.free_pages()

    def pages_held(self, rid) -> int:
        if not self.cache.has_request(rid):
            return 0
        return max((len(t) for t in self.cache.requests[rid].tables.values()), default=0)

    def release(self, rid) -> None:
        if self.cache.has_request(rid):
            self.cache.release(rid)


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


class Scheduler:
    def __init__(self, config: SchedulerConfig, pool: PagePool):
        self.config, self.pool = config, pool
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.finished: List[Sequence] = []
        self._arrivals = itertools.count()
        self.stats = {"steps": 0, "preemptions": 0, "forced": 0, "deferred": 0}

    # -- requests ---------------------------------------------------------------------
    def add_request(self, request_id: Hashable, prompt: Sequence[int], params: SamplingParams,
                    max_positions: int) -> Sequence:
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if len(prompt) >= max_positions:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room below max_position_embeddings={max_positions}")
        # crates/prelude-core/src/engine/model_runner/generate.rs:24-26
        max_new = min(params.max_new_tokens, max_positions - len(prompt))
        seq = Sequence(request_id, list(prompt), params, max_new, next(self._arrivals))
        self.waiting.append(seq)
        return seq

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, request_id: Hashable) -> bool:
        for seq in list(self.waiting):
            if seq.request_id == request_id:
                self.waiting.remove(seq)
                self._finish(seq, "abort")
                return True
        for seq in self.running:
            if seq.request_id == request_id:
                self._finish(seq, "abort")
                return True
        return False

    # -- one scheduling decision ------------------------------------------------------
    def _portion(self, seq: Sequence, budget: int) -> int:
        n = min(seq.pending, budget)
        cap = self.config.long_prefill_token_threshold
        if cap > 0 and seq.prefilling:
            n = min(n, cap)
        return n

    def _pages_for(self, seq: Sequence, upto: int) -> int:
        return max(0, _ceil_div(upto, self.config.page_size) - self.pool.pages_held(seq.request_id))

    def _tokens_in_use(self) -> int:
        return sum(s.total_len for s in self.running)

    def schedule(self) -> List[ScheduledItem]:
        """Decide the next step.  The returned portions are already counted as
        given out; ``on_step_done`` confirms them."""
        cfg = self.config
        self.running = [s for s in self.running if s.status == RUNNING]
        preempted = self._enforce_token_budget()
        budget = cfg.max_num_batched_tokens
        free = self.pool.free_pages()
        items: List[ScheduledItem] = []
        starved: List[Sequence] = []

        # 1. running requests first
        for seq in self.running:
            if budget == 0:
                break
            n = self._portion(seq, budget)
            if n <= 0:
                continue
            need = self._pages_for(seq, seq.computed + n)
            if need > free:
                # shrink a prompt portion to the pages that are left; a single token cannot shrink
                room = (self.pool.pages_held(seq.request_id) + free) * cfg.page_size - seq.computed
                n = min(n, max(0, room))
                need = self._pages_for(seq, seq.computed + n) if n > 0 else 0
            if n <= 0:
                starved.append(seq)
                self.stats["deferred"] += 1
                continue
            free -= need
            budget -= n
            items.append(ScheduledItem(seq, n, seq.computed))

        # 2. waiting requests
        if not preempted and budget > 0 and not self._short_decode_tail(items):
            reserved = sum(self._pages_for(s, s.total_len) for s in self.running if s.prefilling)
            scheduled_growth = sum(self._pages_for(it.seq, it.start + it.n_tokens) for it in items if it.seq.prefilling)
            reserved = max(0, reserved - scheduled_growth)
            slots = cfg.max_running_requests - len(self.running)
            while self.waiting and slots > 0 and budget > 0:
                seq = self.waiting[0]
                footprint = seq.total_len + min(seq.remaining_new, cfg.decode_reservation_cap)
                if cfg.max_total_tokens and self._tokens_in_use() + seq.total_len > cfg.max_total_tokens and self.running:
                    break
                if _ceil_div(footprint, cfg.page_size) + reserved > free:
                    break
                n = self._portion(seq, budget)
                if n <= 0:
                    break
                self.waiting.popleft()
                seq.status = RUNNING
                self.running.append(seq)
                first_pages = _ceil_div(n, cfg.page_size)
                free -= first_pages
                reserved += _ceil_div(seq.total_len, cfg.page_size) - first_pages
                budget -= n
                slots -= 1
                items.append(ScheduledItem(seq, n, 0))

        # 3. nothing fits: force progress
        if not items:
            items = self._force_progress(starved)

        for it in items:
            it.seq.scheduled = it.n_tokens
        if items:
            self.stats["steps"] += 1
        return items

    def _short_decode_tail(self, items: List[ScheduledItem]) -> bool:
        """Every decoding request of the step is within a few tokens of its end
        (crates/prelude-core/src/scheduler/admission.rs:196-208)."""
        limit = self.config.decode_priority_max_remaining_tokens
        decodes = [it.seq for it in items if not it.seq.prefilling]
        if limit == 0 or not decodes:
            return False
        return all(s.remaining_new <= limit for s in decodes)

    def _enforce_token_budget(self) -> bool:
        """Keep the tokens held by running requests within ``max_total_tokens``
        by preempting the newest (preemption.rs:34-73)."""
        limit = self.config.max_total_tokens
        if not limit:
            return False
        preempted = False
        while len(self.running) > 1 and self._tokens_in_use() + len(self.running) > limit:
            victim = max(self.running, key=lambda s: s.arrival)
            self._preempt(victim)
            preempted = True
        return preempted

    def _force_progress(self, starved: List[Sequence]) -> List[ScheduledItem]:
        cfg = self.config
        if starved:
            # running requests exist but none can get a page
            if len(self.running) > 1:
                oldest = min(self.running, key=lambda s: s.arrival)
                victim = max((s for s in self.running if s is not oldest), key=lambda s: (s.preempt_count, s.arrival))
                self._preempt(victim)
                return self.schedule()
            lone = self.running[0]
            self._finish(lone, "cache_full")
            return self.schedule() if self.has_work() else []
        if self.waiting and not self.running:
            seq = self.waiting[0]
            free = self.pool.free_pages()
            if free * cfg.page_size < seq.total_len:
                # the pool cannot hold this request even when it is alone
                self.waiting.popleft()
                self._finish(seq, "cache_full")
                return self.schedule() if self.has_work() else []
            # the reservation for generated tokens did not fit: admit anyway, one token at least
            self.waiting.popleft()
            seq.status = RUNNING
            self.running.append(seq)
            n = max(1, min(self._portion(seq, cfg.max_num_batched_tokens), free * cfg.page_size))
            self.stats["forced"] += 1
            return [ScheduledItem(seq, n, 0)]
        return []

    def _preempt(self, victim: Sequence) -> None:
        self.running.remove(victim)
        self.pool.release(victim.request_id)
        victim.status = WAITING
        victim.computed = 0
        victim.scheduled = 0
        victim.preempt_count += 1
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1

    # -- after the step -----------------------------------------------------------------
    def on_step_done(self, item: ScheduledItem, token: Optional[int], eos_token_ids: Sequence[int] = ()) -> None:
        """Confirm a portion; ``token`` is the sampled token when the portion
        reached the request's end (``item.samples``), else None."""
        seq = item.seq
        if seq.status != RUNNING:
            return
        seq.computed += item.n_tokens
        seq.scheduled = 0
        if token is None:
            return
        seq.output.append(int(token))
        # stop checks in the reference's order: end-of-sequence, stop tokens, length
        # (crates/prelude-core/src/engine/run/ar.rs:1546-1577)
        if not seq.params.ignore_eos and int(token) in eos_token_ids:
            self._finish(seq, "eos")
        elif int(token) in seq.params.stop_token_ids:
            self._finish(seq, "stop")
        elif len(seq.output) >= seq.max_new_tokens:
            self._finish(seq, "length")

    def rollback(self, item: ScheduledItem) -> None:
        """The step could not run this portion after all: nothing is confirmed."""
        item.seq.scheduled = 0

    def _finish(self, seq: Sequence, reason: str) -> None:
        seq.status = FINISHED
        seq.finish_reason = reason
        if seq in self.running:
            self.running.remove(seq)
        self.pool.release(seq.request_id)
        self.finished.append(seq)

    def drain_finished(self) -> List[Sequence]:
        out, self.finished = self.finished, []
        return out
