"""Command line: ``prelude --model <dir> --prompt-ids 1,2,3 ...``.

The engine options carry the names, meanings and defaults of the reference's
command line (crates/prelude-server/src/main.rs:15-183) and of its environment
variables (crates/prelude-core/src/config.rs:114-255); what belongs to its HTTP
server (--host, --port, --api-key, --cors-allow-origin, --pseudo, --task,
--moe-backend, --deltanet-pool-slots, --max-batch-size, --max-batch-wait-ms)
has no meaning here and is not offered.  Prompts are token ids: the tokenizer
is outside this engine.  One JSON object per request is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional, Sequence


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ[name])
    except (KeyError, ValueError):
        return default


def _env_float(name: str, default: float) -> float:
    try:
        return float(os.environ[name])
    except (KeyError, ValueError):
        return default


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="prelude", description="Generate tokens with a model folder on one B200.")
    ap.add_argument("--model", "--model-path", dest="model", required=True,
                    help="Local path to model directory (config.json + safetensors)")
    ap.add_argument("--dtype", default="bf16", choices=["f32", "bf16", "float32", "bfloat16"],
                    help="Override dtype: f32 or bf16 (default bf16)")
    ap.add_argument("--device", default=os.environ.get("PRELUDE_DEVICE", "auto"),
                    help="Device: auto, cuda, cuda:N (there is no cpu path; env PRELUDE_DEVICE)")
    ap.add_argument("--max-running-requests", type=int, default=256, help="Max concurrent running requests in scheduler")
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192,
                    help="Per-step total token budget (prefill + decode combined)")
    ap.add_argument("--long-prefill-token-threshold", type=int, default=0,
                    help="Per-request prefill token cap (0 = no cap, only limited by per-step budget)")
    ap.add_argument("--max-total-tokens", type=int, default=0,
                    help="Max total tokens across all running requests. 0 = bounded by the cache pages only")
    ap.add_argument("--decode-reservation-cap", type=int, default=0,
                    help="Per-request cap for reserving future decode tokens in the scheduler. "
                         "0 = read model's max_position_embeddings")
    ap.add_argument("--decode-priority-max-remaining-tokens", type=int, default=4,
                    help="Prioritize running decode requests with at most this many tokens remaining before "
                         "admitting new prefill work. 0 disables.")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9,
                    help="Fraction of GPU memory for weights and KV cache (0.0-1.0). "
                         "Ignored when --num-pages or PRELUDE_PAGED_ATTN_BLOCKS is set.")
    ap.add_argument("--chunked-prefill", dest="chunked_prefill", action="store_true", default=True,
                    help="Cut prompts into portions under the per-step token budget, beside decode tokens (default)")
    ap.add_argument("--no-chunked-prefill", dest="chunked_prefill", action="store_false",
                    help="Whole prompts only: the per-step budget is raised to the longest request the model allows")
    ap.add_argument("--decode-burst", type=int, default=8,
                    help="Decode steps queued on the device at a time when nothing can change the batch (1 = off)")
    ap.add_argument("--cuda-graph", dest="cuda_graph", action="store_true", default=True,
                    help="Enable CUDA graph capture for decode steps")
    ap.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false",
                    help="Disable CUDA graph capture for decode steps")
    ap.add_argument("--page-size", type=int, default=_env_int("PRELUDE_PAGED_BLOCK_SIZE", 16),
                    help="Tokens per KV cache page (env PRELUDE_PAGED_BLOCK_SIZE)")
    ap.add_argument("--num-pages", type=int, default=_env_int("PRELUDE_PAGED_ATTN_BLOCKS", 0),
                    help="KV cache pages; 0 = size from --gpu-memory-utilization (env PRELUDE_PAGED_ATTN_BLOCKS)")
    ap.add_argument("--cuda-graph-max-bs", type=int, default=_env_int("PRELUDE_CUDA_GRAPH_MAX_BS", 64),
                    help="Largest decode batch that is captured as a CUDA graph (env PRELUDE_CUDA_GRAPH_MAX_BS)")
    ap.add_argument("--max-model-len", type=int, default=0, help="Cap on a request's length; 0 = max_position_embeddings")
    # the request(s)
    ap.add_argument("--random-weights", action="store_true",
                    help="Read config.json alone from --model and draw the weights from --seed on the device")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="A prompt as comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-file", help="File with one prompt per line: comma- or space-separated token ids")
    ap.add_argument("--max-new-tokens", "--max-tokens", dest="max_new_tokens", type=int,
                    default=_env_int("PRELUDE_DEFAULT_MAX_TOKENS", 4096))
    ap.add_argument("--temperature", type=float, default=_env_float("PRELUDE_DEFAULT_TEMPERATURE", 0.7))
    ap.add_argument("--top-p", type=float, default=_env_float("PRELUDE_DEFAULT_TOP_P", 1.0))
    ap.add_argument("--top-k", type=int, default=0, help="0 = off")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--stop-token-ids", default="", help="Comma-separated token ids that end a request")
    ap.add_argument("--ignore-eos", action="store_true")
    return ap


def _parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    prompts = [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            prompts += [_parse_ids(line) for line in f if line.strip()]
    if not prompts:
        sys.stderr.write("prelude: give at least one prompt with --prompt-ids or --prompt-file\n")
        return 2
    device = args.device
    if device in ("auto", "cuda"):
        device = "cuda:0"
    if device == "cpu":
        sys.stderr.write("prelude: this engine runs on sm_100a GPUs only; there is no cpu path\n")
        return 2
    from .engine import Engine
    from .scheduler import SamplingParams
    try:
        budget = args.max_num_batched_tokens
        if not args.chunked_prefill:
            # a prompt is never cut: the budget must hold the longest request (the reference instead runs
            # prompt-only and decode-only steps in this mode, crates/prelude-core/src/scheduler/admission.rs:211-254)
            from ..config import load_model_config
            with open(os.path.join(args.model, "config.json"), "r", encoding="utf-8") as f:
                limit = load_model_config(json.load(f)).to_model_spec().max_positions
            budget = max(budget, args.max_model_len or limit)
        engine = Engine(args.model, dtype=args.dtype, device=device, page_size=args.page_size,
                        num_pages=args.num_pages or None, gpu_memory_utilization=args.gpu_memory_utilization,
                        max_running_requests=args.max_running_requests,
                        max_num_batched_tokens=budget, decode_burst=args.decode_burst,
                        long_prefill_token_threshold=args.long_prefill_token_threshold,
                        max_total_tokens=args.max_total_tokens, decode_reservation_cap=args.decode_reservation_cap,
                        decode_priority_max_remaining_tokens=args.decode_priority_max_remaining_tokens,
                        cuda_graph=args.cuda_graph, cuda_graph_max_bs=args.cuda_graph_max_bs,
                        max_model_len=args.max_model_len or None,
                        random_weights_seed=args.seed if args.random_weights else None)
        params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k or None,
                                seed=args.seed, max_new_tokens=args.max_new_tokens,
                                stop_token_ids=tuple(_parse_ids(args.stop_token_ids)), ignore_eos=args.ignore_eos)
        results = engine.generate(prompts, params)
    except Exception as e:  # noqa: BLE001 - one line for the user
        sys.stderr.write(f"prelude: {type(e).__name__}: {e}\n")
        return 1
    for r in results:
        print(json.dumps({"request_id": r.request_id, "token_ids": r.token_ids, "finish_reason": r.finish_reason,
                          "usage": {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens},
                          "metrics": {"ttft_ms": round(r.ttft_ms, 3), "total_ms": round(r.total_ms, 3)}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
