"""Command line of the engine.

    python -m sandyrt_b200 generate --model DIR --prompt-ids 1,2,3 [options]
    python -m sandyrt_b200 random-model --config config.json --out DIR [--seed S] [--dtype bfloat16]
    python -m sandyrt_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl

Option names follow the reference's worker where it has them (src/server/SandyWorkerMain.cpp:30-39:
--model, --prefill-chunk-tokens, --eos-token-id, --max-context-tokens, --profile, --debug) and
its request fields (proto/sandy_inference.proto: max_tokens, temperature, top_p, stop ids).
The reference's `--weights` and `--architecture` have no counterpart: a model folder holds its
weights and its config.json names its architecture.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(a) -> int:
    from .engine.llm import LLM

    prompts: List[List[int]] = []
    for p in a.prompt_ids or []:
        prompts.append(_ids(p))
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        print("no prompt: give --prompt-ids or --prompt-file", file=sys.stderr)
        return 1
    llm = LLM(a.model, dtype=a.dtype, cache_tokens=a.cache_tokens, page_size=a.page_size, max_live=a.max_seqs,
              max_step_tokens=a.max_batch_tokens, prefill_chunk_tokens=a.prefill_chunk_tokens,
              eos_token_ids=a.eos_token_id, max_context_tokens=a.max_context_tokens)
    results = llm.generate(prompts, max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p,
                           top_k=a.top_k, seed=a.seed, stop_token_ids=a.stop_id or [], report=a.profile)
    for i, r in enumerate(results):
        print(json.dumps({"request": i, "output_ids": r.output_ids, "finish_reason": r.finish_reason,
                          "prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
                          "prefill_ms": round(r.prefill_ms, 3), "decode_ms": round(r.decode_ms, 3),
                          "prefill_toks_per_s": round(r.prefill_tokens_per_second, 1),
                          "decode_toks_per_s": round(r.decode_tokens_per_second, 1)}))
    if a.debug:
        print(json.dumps({"scheduler": dict(llm.scheduler.stats),
                          "pages_high_water": [p.high_water for p in llm.engine.cache.alloc.pools]}), file=sys.stderr)
    return 0


def cmd_random_model(a) -> int:
    import torch

    from .config.base import architecture_name
    from .registry import get_architecture
    from .weights.random_init import write_random_model

    with open(a.config) as f:
        raw = json.load(f)
    cfg = get_architecture(architecture_name(raw)).config_cls.from_dict(raw)
    out = write_random_model(cfg, a.out, seed=a.seed, dtype={"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype])
    print(out)
    return 0


def cmd_replay(a) -> int:
    from .engine.replay import run

    return run(a.model, a.dtype, a.out, a.max_tokens, sys.stdin, page_size=a.page_size)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="sandyrt_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="generate tokens for one or more prompts of token ids")
    g.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", help="comma- or space-separated ids (repeatable)")
    g.add_argument("--prompt-file", help="one prompt of ids per line")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--seed", type=int, default=None, help="sampling seed")
    g.add_argument("--stop-id", type=int, action="append", help="stop token for these requests (repeatable)")
    g.add_argument("--eos-token-id", type=int, action="append", help="stop token for every request (repeatable)")
    g.add_argument("--prefill-chunk-tokens", "--prefill-chunk-size", type=int, default=2048)
    g.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    g.add_argument("--max-seqs", type=int, default=64, help="most requests live at once")
    g.add_argument("--max-context-tokens", type=int, default=0)
    g.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache pool holds")
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--profile", action="store_true", help="print the throughput line per request")
    g.add_argument("--debug", action="store_true")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random_model)

    t = sub.add_parser("replay", help="feed token ids step by step and write logits (see bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--page-size", type=int, default=16)
    t.set_defaults(fn=cmd_replay)

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
