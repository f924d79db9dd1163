"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing.  It drives the same model, step function, cache manager and kernels that
generation uses (the host library's, through Engine.step); nothing here computes anything about
the model itself.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["b"]}
`entries`: for each request its next tokens and the places among them whose logits are
wanted; all entries of a step run as one batch.  `end`: requests that are finished after
this step; their pages and slot are given back.  For a step with wanted places the logits
are written to `<out>/<step>.f32` as little-endian float32 [wanted, vocab], in the order of
the entries and of `want`.  After every step `done <step>` is printed and flushed.

The reference has nothing equivalent; its closest tool is a greedy generation runner
(test/engine/MultiGemmaRunner.cpp:426-792).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}
MAX_LIVE_REQUESTS = 64


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def run(model_dir: str, dtype_name: str, out_dir: str, max_tokens: int, lines,
        page_size: int = 16, log=sys.stdout) -> int:
    import torch

    from ..models.model import load_model
    from .step import Engine, StepEntry

    if not torch.cuda.is_available():
        raise RuntimeError("trace_run needs a CUDA device; this engine has no CPU path")
    dtype = getattr(torch, DTYPES[dtype_name])
    os.makedirs(out_dir, exist_ok=True)
    model = load_model(model_dir, device="cuda:0", dtype=dtype)
    # The pool holds `max_tokens` tokens, in whole pages.
    engine = Engine(model, max_tokens=_round_up(max_tokens, page_size), page_size=page_size,
                    max_requests=MAX_LIVE_REQUESTS)
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        rec = json.loads(raw)
        step = rec["step"]
        entries: List[StepEntry] = []
        n_want = 0
        for e in rec.get("entries", []):
            toks = [int(t) for t in e.get("tokens", [])]
            want = [int(w) for w in e.get("want", [])]
            if toks:
                entries.append(StepEntry(e["id"], toks, want))
                n_want += len(want)
        if entries:
            logits = engine.step(entries)
            if n_want:
                host = logits.to("cpu", copy=True).contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f"{step}.f32.tmp")
                host.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
            engine.check_status()
        for rid in rec.get("end", []):
            if rid in engine.cache.alloc:
                engine.release(rid)
        print(f"done {step}", file=log, flush=True)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the cache pool)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (power of two)")
    args = ap.parse_args(argv)
    return run(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, page_size=args.page_size)


if __name__ == "__main__":
    sys.exit(main())
