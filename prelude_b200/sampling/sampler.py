"""Choosing the next token of every request that reached its last position.

Greedy and plain temperature sampling run on the device in one kernel for the
whole batch.  Requests that ask for top-k or top-p take the reference's route
(crates/prelude-core/src/engine/sampling/logits_processor.rs:44-135): the
softmax at their temperature is computed on the device, the probabilities come
to the host, the filter is applied there and the token is drawn there.

Which sampler a request gets follows ``build_sampling``
(crates/prelude-core/src/engine/model_runner/postprocess.rs:18-38): temperature
below 1e-7 is greedy; a positive top_k means top-k then top-p; top_p below 1
means top-p; else the whole distribution.

Randomness: one Philox4x32-10 number per drawn token, keyed by the request's
seed with the count of tokens the request has generated so far as counter, so
a request's tokens do not depend on what else is in the batch.  (The reference
draws from a host generator seeded per request; its stream is not reproduced.)
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..ops import kernels as K

GREEDY_BELOW = 1e-7


def sampling_mode(temperature: float, top_k, top_p: float) -> str:
    if temperature < GREEDY_BELOW:
        return "greedy"
    if top_k is not None and top_k > 0:
        return "top_k_top_p"
    if top_p < 1.0:
        return "top_p"
    return "all"


def filter_top_p(probs: np.ndarray, top_p: float) -> np.ndarray:
    """Sort descending, keep tokens until the running sum reaches top_p, zero the rest
    (logits_processor.rs:51-63): a token stays if the sum of those before it, in that order, is below top_p."""
    order = np.argsort(-probs, kind="stable")
    sorted_probs = probs[order].astype(np.float64)
    before = np.cumsum(sorted_probs) - sorted_probs
    out = probs.copy()
    out[order[before >= top_p]] = 0.0
    return out


def filter_top_k(probs: np.ndarray, top_k: int) -> np.ndarray:
    """Keep the k most probable tokens (logits_processor.rs:65-94)."""
    if top_k >= probs.shape[0]:
        return probs
    keep = np.argsort(-probs, kind="stable")[:top_k]
    out = np.zeros_like(probs)
    out[keep] = probs[keep]
    return out


def draw(probs: np.ndarray, u: float) -> int:
    """First index whose cumulative weight, in index order, exceeds u * total."""
    cum = np.cumsum(probs.astype(np.float64))
    total = cum[-1]
    if not total > 0:
        return int(np.argmax(probs))
    idx = int(np.searchsorted(cum, u * total, side="right"))
    idx = min(idx, probs.shape[0] - 1)
    while probs[idx] == 0 and idx > 0:       # rounding at the far end
        idx -= 1
    return idx


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], top_ks: Sequence, top_ps: Sequence[float],
               seeds: Sequence[int], counters: Sequence[int]) -> List[int]:
        """One token per row of ``logits`` ([rows, vocab] float32 on the device)."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        modes = [sampling_mode(t, k, p) for t, k, p in zip(temperatures, top_ks, top_ps)]
        if all(m == "greedy" for m in modes):
            return K.argmax(logits).tolist()
        meta = np.zeros((3, rows), dtype=np.int64)
        meta[0] = np.asarray([np.float32(t).view(np.int32) for t in temperatures], dtype=np.int64)
        meta[1] = np.asarray([s & (2**63 - 1) for s in seeds], dtype=np.int64)
        meta[2] = np.asarray(counters, dtype=np.int64)
        dev = torch.from_numpy(meta).to(self.device, non_blocking=True)
        temps = dev[0].to(torch.int32).view(torch.float32)
        tokens = K.sample(logits, temps, dev[1].contiguous(), dev[2].contiguous())
        host_rows = [i for i, m in enumerate(modes) if m in ("top_p", "top_k_top_p")]
        if not host_rows:
            return tokens.tolist()
        idx = torch.as_tensor(host_rows, dtype=torch.long, device=self.device)
        probs = K.softmax_temperature(logits.index_select(0, idx).contiguous(), temps.index_select(0, idx).contiguous())
        probs = probs.cpu().numpy()
        out = tokens.tolist()
        for j, i in enumerate(host_rows):
            p = probs[j]
            if modes[i] == "top_k_top_p":
                p = filter_top_k(p, int(top_ks[i]))
                if 0.0 < top_ps[i] < float(p.sum()):
                    p = filter_top_p(p, float(top_ps[i]))
            elif 0.0 < top_ps[i] < 1.0:
                p = filter_top_p(p, float(top_ps[i]))
            out[i] = draw(p, K.philox_uniform(int(seeds[i]), int(counters[i])))
        return out
