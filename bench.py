"""Benchmark of the engine: decode tokens per second, prefill tokens per second, rooflines.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: GPT-2 small (12 layers, width 768, 12 heads of 64, inner 3072, vocabulary
50257, 1024 positions) with seeded random weights in bfloat16, a batch of 8 requests with
128-token prompts of uniform random ids; one "step" is one decode step of the whole batch.
Prints ONE JSON line.  `value` is decoded tokens per second timed on the device over K
steps; `e2e` is the same through the Python entry point (LLM.add_request/step: host token
ids in, every step's drawn tokens read back to the host); `prefill` is one step over 2,048
prompt tokens (2 prompts x 1,024); `roofline` relates the decode step to HBM bandwidth;
`points` holds decode tokens per second at batch 1 and 64.

The engine runs on one GPU: for --gpus N > 1 it prints one line that says so and exits 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# GPT-2 small: experiments/gpt2_small/config.json of the reference
SMALL = dict(n_layer=12, n_embd=768, n_head=12, n_positions=1024, vocab_size=50257, n_inner=3072,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(float(p[0])); mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    """The reference cannot run this metric: its GPT-2 is a fixed 16-token, CPU-only forward
    with no cache, no decode loop and no sampler (src/models/gpt2_small.sandy.go:47-59,
    scripts/run_gpt2.py:17,334-336), and its CUDA device has no linear kernel
    (src/device/cuda/CudaDevice.cpp:536-537)."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference has no GPT-2 decode path (fixed 16-token CPU-only forward, no KV cache, no "
                      "sampler; its CUDA backend lacks the linear kernel) and it is a CMake project with no "
                      "Python package to pip-install"}))
    return 0


def make_model(n_layer: int, seed: int = 0):
    import torch

    from sandyrt_b200.config.gpt2 import GPT2Config
    from sandyrt_b200.models.model import build_model, describe
    from sandyrt_b200.weights.random_init import random_tensors

    cfg = GPT2Config(**{**SMALL, "n_layer": n_layer})
    cfg.validate()
    model = build_model(describe(cfg))
    tensors = random_tensors(model.tensor_requests(), seed, torch.bfloat16)
    model.bind(tensors, "cuda:0", torch.bfloat16)
    model.config = cfg
    return model, cfg


def _start_decoding(llm, batch, prompt_len, max_tokens, warmup, rng, vocab):
    """Add `batch` requests, run their prompts and `warmup` decode steps through the entry point."""
    rids = [llm.add_request(rng.integers(0, vocab, size=prompt_len).tolist(), max_tokens=max_tokens)
            for _ in range(batch)]
    while any(len(llm._requests[r].output) == 0 for r in rids):       # prefill
        llm.step()
    for _ in range(warmup):
        llm.step()
    return rids


def _drop(llm, rids):
    for r in rids:
        llm.abort(r)
    llm.drain()
    for r in rids:
        llm.forget(r)


def decode_run(llm, batch, prompt_len, steps, warmup, rng, vocab, want_e2e=True):
    """Times `steps` decode steps of `batch` requests after `warmup` untimed ones, twice:

    device: the engine's decode bursts (a burst's index arrays, block tables and sampling options
            copied from pinned memory; per step the model and the sampler, which feeds the drawn
            token to the next step on the device), bursts queued back to back with no read-back
            in between, timed with CUDA events;
    e2e:    the same number of steps through the entry point (LLM.step: scheduler, bursts of
            decode steps with the drawn tokens of every step read back to the host), timed on
            the wall clock.

    Returns (device ms/step, (e2e ms/step, host-to-device and device-to-host bytes per step of that
    loop), mean context length, launches per step)."""
    import numpy as np
    import torch

    from sandyrt_b200.engine.step import SampleRow, StepEntry

    e2e_ms, e2e_h2d, e2e_d2h = None, 0.0, 0.0
    if want_e2e:
        rids = _start_decoding(llm, batch, prompt_len, steps + 10 * warmup + 80, warmup, rng, vocab)
        torch.cuda.synchronize()
        first = llm.decode_steps_run
        h2d0, d2h0 = llm.engine.h2d_bytes_total, llm.engine.d2h_bytes_total
        t0 = time.perf_counter()
        while llm.decode_steps_run - first < steps:     # a call may run a burst of several steps
            llm.step()
        llm.drain()                                     # a burst queued ahead: its steps count, and so does its time
        torch.cuda.synchronize()
        n_steps = llm.decode_steps_run - first
        e2e_ms = (time.perf_counter() - t0) * 1e3 / n_steps
        e2e_h2d = (llm.engine.h2d_bytes_total - h2d0) / n_steps
        e2e_d2h = (llm.engine.d2h_bytes_total - d2h0) / n_steps
        _drop(llm, rids)

    rids = _start_decoding(llm, batch, prompt_len, 100000, warmup, rng, vocab)
    llm.drain()                                          # the loop below drives the engine itself
    engine = llm.engine
    ctx0 = sum(engine.length(r) for r in rids) / batch
    rows = [SampleRow() for _ in rids]
    burst = llm.max_burst
    first = [int(t) for t in rng.integers(0, vocab, size=batch)]

    def queue(n, in_flight):
        """n more decode steps of all requests, queued behind the in_flight steps already queued."""
        entries = [StepEntry(r, [0 if in_flight else first[k]], [0]) for k, r in enumerate(rids)]
        return engine.decode_burst_async(entries, rows, np.zeros((n, batch), dtype=np.float32), in_flight=in_flight)

    # untimed (the entry point's warm-up above has already made the engine record this burst shape)
    in_flight = 0
    for _ in range(2):
        queue(burst, in_flight)
        in_flight += burst
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    done = 0
    while done < steps:
        n = min(burst, steps - done)
        last = queue(n, in_flight)
        in_flight += n
        done += n
    e1.record()
    torch.cuda.synchronize()
    if (engine.burst_tokens(last) < 0).any():
        raise RuntimeError("the sampler reported bad logits")
    engine.check_status()
    dev_ms = e0.elapsed_time(e1) / steps
    for r in rids:
        engine.commit(r, engine.length(r) + in_flight)
    ctx1 = sum(engine.length(r) for r in rids) / batch
    launches = engine.last_launches
    _drop(llm, rids)
    return dev_ms, (e2e_ms, e2e_h2d, e2e_d2h), 0.5 * (ctx0 + ctx1), launches


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--layers", type=int, default=SMALL["n_layer"])
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from sandyrt_b200.engine.llm import LLM
    from sandyrt_b200.engine.step import StepEntry

    peaks = load_peaks()
    model, cfg = make_model(args.layers)
    vocab = cfg.vocab_size
    rng = np.random.default_rng(0)
    llm = LLM(model, cache_tokens=64 * 1024 + 4096, max_live=64, max_step_tokens=4096, prefill_chunk_tokens=2048)
    engine = llm.engine

    clocks = ClockSampler()
    clocks.start()

    # ---- decode at the headline batch: device-timed step of the engine + sampler ------------
    # The same loop gives the end-to-end number through the entry point.  While all requests are
    # decoding, llm.step() runs bursts of up to 8 decode steps: a burst's index arrays, block
    # tables and sampling options are packed into pinned memory and copied to the device, the
    # sampler feeds each drawn token to the next step on the device, and every step's drawn
    # tokens are copied back to pinned memory and handed to the scheduler; the next burst is
    # queued before the last one's tokens are read.  The byte counts are those copies, per step.
    dev_ms, (wall_ms, e2e_h2d, e2e_d2h), mean_ctx, launches_per_step = decode_run(llm, args.batch, args.prompt_len, args.steps,
                                                              args.warmup, rng, vocab)
    value = args.batch / (dev_ms / 1e3)
    e2e_value = args.batch / (wall_ms / 1e3)
    weight_bytes = model.weight_bytes()
    kv_bytes = engine.cache.kv_bytes_per_token() * args.batch * mean_ctx
    achieved_gbs = (weight_bytes + kv_bytes) / (dev_ms / 1e3) / 1e9

    # ---- prefill of 2,048 tokens: 2 prompts x 1,024 in one step ------------------------------
    T = 2048
    prompts = [rng.integers(0, vocab, size=1024).tolist() for _ in range(2)]
    prefill_ms = []
    for it in range(3 + 5):
        entries = [StepEntry(f"p{it}-{i}", p, [len(p) - 1]) for i, p in enumerate(prompts)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step(entries)
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            prefill_ms.append(e0.elapsed_time(e1))
        for e in entries:
            engine.release(e.rid)
    pf_ms = sorted(prefill_ms)[len(prefill_ms) // 2]
    E, I, L, V = cfg.n_embd, cfg.inner_dim, cfg.n_layer, cfg.vocab_size
    gemm_flops = 2.0 * T * L * (E * 3 * E + E * E + 2 * E * I) + 2.0 * 2 * E * V
    attn_flops = L * 2 * (2.0 * 2 * E * (1024 * 1025 / 2))      # QK^T and PV over the causal half, 2 prompts
    pf_flops = gemm_flops + attn_flops
    pf_frac = pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            d_ms, _, _, _ = decode_run(llm, b, args.prompt_len, min(args.steps, 128), args.warmup, rng, vocab,
                                       want_e2e=False)
            points[f"decode_b{b}"] = b / (d_ms / 1e3)

    clock_info = clocks.stop()
    launches = launches_per_step * args.steps
    out = {
        "metric": "decode tok/s at batch 8 (GPT-2 small)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "gpt2-small", "n_layer": cfg.n_layer, "n_layer_full": SMALL["n_layer"], "n_embd": E,
                   "n_head": cfg.n_head, "head_dim": cfg.head_dim, "n_inner": I, "vocab_size": V,
                   "n_positions": cfg.n_positions, "global_batch": args.batch, "seq_len": cfg.n_positions,
                   "prompt_len": args.prompt_len, "mean_context": round(mean_ctx, 1), "page_size": engine.cache.page_size,
                   "parallelism": "single-gpu", "weights": "random seed 0",
                   "l2": "inputs larger than L2 (weights %.0f MB)" % (weight_bytes / 1e6)},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": wall_ms,
                "h2d_bytes_per_step": round(e2e_h2d, 1), "d2h_bytes_per_step": round(e2e_d2h, 1),
                "steps_per_burst": llm.max_burst, "bursts_queued_ahead": bool(llm.pipeline_bursts)},
        "gpu_launches": launches,
        "prefill": {"value": T / (pf_ms / 1e3), "tokens": T, "ms": pf_ms, "frac": pf_frac,
                    "peak": f"{peaks['bf16_tflops']} TFLOP/s bf16 of {peaks['source']}"},
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"], "of": peaks["source"],
                     "bytes_per_step": weight_bytes + kv_bytes},
        "points": points,
        "clocks": clock_info,
    }
    print(f"[bench] graph replays {engine.graph_replays}, recorded graphs {len(engine._graphs)}, "
          f"stale graphs dropped {engine.stale_graphs}", file=sys.stderr)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
