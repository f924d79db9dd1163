"""Command line of the engine.

    python -m sandyrt_b200 generate --model DIR --prompt-ids 1,2,3 [options]
    python -m sandyrt_b200 random-model --config config.json --out DIR [--seed S] [--dtype bfloat16]
    python -m sandyrt_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl
    python -m sandyrt_b200 program-timeline --model DIR [--batch 8] [--context 300]

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


def cmd_program_timeline(a) -> int:
    """Run decode steps of `batch` requests at about `context` tokens as a decode program and print
    where block 0 spent the time of one launch, operation by operation."""
    import numpy as np
    import torch

    from .engine.step import Engine, StepEntry
    from .models.model import load_model

    model = load_model(a.model, device="cuda:0", dtype=torch.bfloat16)
    eng = Engine(model, max_tokens=a.batch * (a.context + 64) + 1024, max_requests=max(a.batch, 1),
                 max_step_tokens=max(2048, a.context), use_cuda_graphs=False, use_decode_programs=True)
    rng = np.random.default_rng(0)
    vocab = model.spec.vocab_size
    for i in range(a.batch):
        eng.step([StepEntry(i, rng.integers(0, vocab, size=a.context).tolist(), [])])
    for _ in range(4):
        eng.step([StepEntry(i, [int(rng.integers(0, vocab))], [0]) for i in range(a.batch)])
    hits = [h for h in eng._programs.values() if h is not None]
    if not hits:
        print("this model's decode step cannot be recorded as a program", file=sys.stderr)
        return 1
    prog = hits[-1][0]
    tl = torch.zeros(3 * prog.n_ops + 1, dtype=torch.int64, device="cuda:0")
    for _ in range(3):      # the last run is the one read: same inputs, caches warm
        prog.run(tl)
        torch.cuda.synchronize()
    eng.check_status()
    t = tl.cpu().numpy().astype(np.int64)
    names = {0: "embed", 1: "norm", 2: "gemm", 3: "attn"}
    print(f"{prog.n_ops} operations, {(t[-1] - t[0]) / 1e3:.1f} us on block 0's clock")
    print(" op kind    total   staged    work  barrier   (us; staged: inputs in shared memory / first keys asked for)")
    total = {}
    for i in range(prog.n_ops):
        s0, m0, m1, end = t[3 * i], t[1 + 3 * i], t[2 + 3 * i], t[3 + 3 * i]
        staged = (m0 - s0) / 1e3 if m0 else 0.0
        work = (m1 - (m0 if m0 else s0)) / 1e3
        kind = names[prog.kinds[i]]
        total[kind] = total.get(kind, 0.0) + (end - s0) / 1e3
        print(f"{i:3d} {kind:5s} {(end - s0) / 1e3:7.2f} {staged:8.2f} {work:7.2f} {(end - m1) / 1e3:8.2f}")
    print("by kind:", ", ".join(f"{k} {v:.1f} us" for k, v in total.items()))
    return 0


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

    pt = sub.add_parser("program-timeline", help="time a decode step run as one resident kernel, operation by operation")
    pt.add_argument("--model", required=True)
    pt.add_argument("--batch", type=int, default=8)
    pt.add_argument("--context", type=int, default=300)
    pt.set_defaults(fn=cmd_program_timeline)

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
