"""Ways of cutting requests into steps, and running them through the engine.

A *schedule* is a list of steps; a step is (entries, ended) with entries a list
of (request id, tokens, wanted places).  ``run_schedule`` feeds a schedule to a
ModelRunner and returns the logits row of every (request, position) asked for.
"""
import random
from typing import Dict, List, Sequence, Tuple

import torch

from prelude_b200.engine.runner import StepEntry


def whole(reqs: Dict[str, List[int]]):
    """Each request alone, the whole prompt in one step."""
    return [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in reqs.items()]


def tail_decode(reqs: Dict[str, List[int]], tail: int = 32):
    """All but the last ``tail`` tokens in one step, then one token a step."""
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append(([(rid, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(rid, toks[i:i + 1], [0])], [rid] if i == len(toks) - 1 else []))
        if head == len(toks):
            steps[-1] = (steps[-1][0], [rid])
    return steps


def portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 16, 3, 2, 5, 11, 2, 1, 4)):
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    for rid, toks in reqs.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            last = i + n == len(toks)
            steps.append(([(rid, toks[i:i + n], list(range(n)))], [rid] if last else []))
            i += n
    return steps


def mixed(reqs: Dict[str, List[int]], max_live: int = 4, seed: int = 0, decode_tail: int = 6):
    """Up to ``max_live`` requests at a time: portions of some beside single
    tokens of others; a request may sit out a step; ended requests make room
    for the next."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            toks = reqs[rid]
            fed = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # sits this step out
            left = len(toks) - fed
            if left <= decode_tail:
                n = 1
            else:
                n = min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 17]))
            entries.append((rid, toks[fed:fed + n], list(range(n))))
            live[rid] = fed + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, ended))
    return steps


def run_schedule(runner, schedule) -> Dict[Tuple[str, int], torch.Tensor]:
    out = {}
    fed: Dict[str, int] = {}
    for entries, ended in schedule:
        logits = runner.step([StepEntry(rid, toks, want) for rid, toks, want in entries]).float().cpu()
        row = 0
        for rid, toks, want in entries:
            base = fed.get(rid, 0)
            for w in want:
                out[(rid, base + w)] = logits[row]
                row += 1
            fed[rid] = base + len(toks)
        assert row == logits.shape[0]
        for rid in ended:
            runner.finish(rid)
            fed.pop(rid, None)
    return out


def peak_tokens(schedule, page_size: int) -> int:
    """Most tokens held at any time, each request rounded up to whole pages."""
    fed: Dict[str, int] = {}
    peak = 0
    for entries, ended in schedule:
        for rid, toks, _ in entries:
            fed[rid] = fed.get(rid, 0) + len(toks)
        peak = max(peak, sum(-(-n // page_size) * page_size for n in fed.values()))
        for rid in ended:
            fed.pop(rid, None)
    return peak
