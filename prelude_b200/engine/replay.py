"""Trace replay: feed given token ids through a model step by step, write logits.

It samples nothing.  It drives the same model, step function, cache and kernels
that generation uses; it has no forward pass, cache or loader of its own.

Standard input holds one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  A request's position is the number of its
tokens fed so far.  For a step in which something is wanted the logits at the
wanted places are written to ``<out>/<step>.f32`` as little-endian float32
[wanted, vocab], in the order of the entries and of ``want``.  Requests named in
``end`` are finished after the step and what they hold is given back.  After
every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence

from .loading import load_model, make_runner
from .runner import StepEntry


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines, page_size: int = 16,
           device: str = "cuda:0", say=print) -> int:
    """Run the steps that ``lines`` yields; returns the number of steps run."""
    import numpy as np

    os.makedirs(out_dir, exist_ok=True)
    model = load_model(model_dir, dtype, device)
    # every live request's count is rounded up to a multiple of 64 by the caller; pages divide 64
    runner = make_runner(model, page_size=page_size, num_pages=max(1, -(-max_tokens // page_size)), max_slots=64,
                         max_request_tokens=max_tokens)
    runner.enable_step_graphs()               # as generation runs them: steps with prompt tokens replay captured pieces
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                       for e in rec.get("entries", [])]
            ended = list(rec.get("end", []))
        except (ValueError, KeyError, TypeError) as e:
            raise ValueError(f"bad trace line {line[:200]!r}: {e}") from None
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in ended:
            if runner.cache.has_request(rid):
                runner.finish(rid)
        say(f"done {step}")
        n += 1
    return n


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (must divide 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size <= 0 or 64 % args.page_size:
        ap.error("--page-size must divide 64")
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")

    def say(msg: str) -> None:
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    try:
        replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, args.page_size, args.device, say)
    except Exception as e:  # noqa: BLE001 - one line for the user, non-zero exit
        sys.stderr.write(f"trace_run: {type(e).__name__}: {e}\n")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
