"""Benchmark of the engine: decode tokens per second, prefill tokens per second, rooflines.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload medium|xl          the mixed-batch workloads through LLM.generate
    python bench.py --profile-kernels             time per kernel class of a decode and a prompt step
    python bench.py --attribute [--batch B]       what each family of launches costs inside a step (leave-one-out)
    python bench.py --micro gemm|decode-attention|prefill-attention [...]   kernel micro-benchmarks

Default workload: GPT-2 small (12 layers, width 768, 12 heads of 64, inner 3072, vocabulary 50257,
1024 positions) with seeded random weights in bfloat16, a batch of 8 requests with 128-token prompts
of uniform random ids; one "step" is one decode step of the whole batch.  Prints ONE JSON line.
`value` is decoded tokens per second timed on the device over K steps (CUDA events on the engine's
stream around bursts queued behind bursts that are still running); `e2e` is the same through the
Python entry point (LLM.add_request/step: host token ids in, every step's drawn tokens read back to
the host), on the wall clock; `prefill` is one step over 2,048 prompt tokens (2 prompts x 1,024);
`roofline` relates the decode step to HBM bandwidth; `points` holds decode at batch 1 and 64, each
with its context, step time and roofline fraction; `fp32` holds the float32 path's decode at batch
1 and 8 and its prefill.

The engine runs on one GPU: for --gpus N > 1 it prints one line that says so and exits 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

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


def load_model_config(name: str) -> dict:
    """configs/gpt2_<name>.json: the config.json of the named size."""
    with open(os.path.join(ROOT, "configs", f"gpt2_{name}.json")) as f:
        return json.load(f)


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


def make_model(raw_config: dict, n_layer: int, dtype_name: str, seed: int = 0):
    """A model of the named configuration (with n_layer layers) with seeded random weights."""
    import torch

    from sandyrt_b200.config.gpt2 import GPT2Config
    from sandyrt_b200.models.model import build_model

    cfg = GPT2Config.from_dict({**raw_config, "n_layer": n_layer})
    cfg.validate()
    model = build_model(cfg)
    model.bind_random(seed, getattr(torch, dtype_name))
    return model, cfg


def _start_decoding(llm, batch, prompt_len, max_tokens, warmup, rng, vocab):
    """Add `batch` requests, run their prompts and `warmup` decode steps through the entry point."""
    rids = [llm.add_request(rng.integers(0, vocab, size=prompt_len).tolist(), max_tokens=max_tokens)
            for _ in range(batch)]
    seen = set()
    while len(seen) < batch:                                          # prefill
        seen.update(r for r, _ in llm.step())
    for _ in range(warmup):
        llm.step()
    return rids


def _drop(llm, rids):
    for r in rids:
        llm.abort(r)
    llm.drain()
    for r in rids:
        llm.forget(r)


MEAN_CONTEXT = 384      # 128-token prompts + 512 generated tokens: the requests' mean length while they decode


def _advance_to(llm, rids, context):
    """Untimed decode steps through the entry point until the requests hold `context` tokens."""
    while llm.engine.length(rids[0]) < context:
        llm.step()
    llm.drain()


def decode_run(llm, batch, prompt_len, steps, warmup, rng, vocab, want_e2e=True):
    """Times `steps` decode steps of `batch` requests after `warmup` untimed ones, twice:

    e2e:    through the entry point (LLM.step: scheduler, bursts of decode steps with the drawn
            tokens of every step read back to the host), timed on the wall clock;
    device: the engine's decode bursts (a burst's index arrays, block tables and sampling options
            copied from pinned memory; per step the model and the sampler, which feeds the drawn
            token to the next step on the device), queued back to back with no read-back in
            between.  Two untimed bursts are queued first and the first event is recorded BEHIND
            them, so the timed bursts are queued while the device is still busy: what is between
            the two events is device work only.

    Both loops time the steps around a context of MEAN_CONTEXT tokens (untimed decode steps bring
    the requests there first), since a decode step's time grows with the keys it reads.

    Returns (device ms/step, (e2e ms/step, host-to-device and device-to-host bytes per step of that
    loop), mean context length of the device loop, launches per step)."""
    import numpy as np

    from sandyrt_b200.engine.step import SampleRow, StepEntry

    e2e_ms, e2e_h2d, e2e_d2h = None, 0.0, 0.0
    engine = llm.engine
    burst = llm.max_burst
    start_context = max(prompt_len + 1, MEAN_CONTEXT - steps // 2)
    if want_e2e:
        rids = _start_decoding(llm, batch, prompt_len, 100000, warmup, rng, vocab)
        _advance_to(llm, rids, start_context)
        engine.synchronize()
        first = llm.decode_steps_run
        h2d0, d2h0 = engine.h2d_bytes_total, engine.d2h_bytes_total
        t0 = time.perf_counter()
        n_steps = 0
        while n_steps < steps:                          # a call may run a burst of several steps
            n_steps += len(llm.step()) // batch
        n_steps += len(llm.drain()) // batch            # a burst queued ahead: its steps count, and so does its time
        engine.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / n_steps
        assert llm.decode_steps_run - first == n_steps
        e2e_h2d = (engine.h2d_bytes_total - h2d0) / n_steps
        e2e_d2h = (engine.d2h_bytes_total - d2h0) / n_steps
        _drop(llm, rids)

    rids = _start_decoding(llm, batch, prompt_len, 100000, warmup, rng, vocab)
    _advance_to(llm, rids, start_context - 2 * burst)    # the loop below drives the engine itself
    ctx0 = sum(engine.length(r) for r in rids) / batch
    rows = [SampleRow() for _ in rids]
    first = [int(t) for t in rng.integers(0, vocab, size=batch)]

    def queue(n, in_flight):
        """n more decode steps of all requests, queued behind the in_flight steps already queued."""
        entries = [StepEntry(r, [0 if in_flight else first[k]], [0]) for k, r in enumerate(rids)]
        return engine.decode_burst_async(entries, rows, np.zeros((n, batch), dtype=np.float32), in_flight=in_flight)

    # untimed (the entry point's steps above have already made the engine record this burst shape);
    # these keep the device busy while the timed ones are queued
    in_flight = 0
    for _ in range(2):
        queue(burst, in_flight)
        in_flight += burst
    before = in_flight
    engine.mark(0)
    done = 0
    while done < steps:
        n = min(burst, steps - done)
        last = queue(n, in_flight)
        in_flight += n
        done += n
    engine.mark(1)
    dev_ms = engine.elapsed_ms() / steps
    if (engine.burst_tokens(last) < 0).any():
        raise RuntimeError("the sampler reported bad logits")
    engine.check_status()
    for r in rids:
        engine.commit(r, engine.length(r) + in_flight)
    mean_ctx = ctx0 + before + 0.5 * steps               # the context of the timed steps
    launches = engine.last_launches
    _drop(llm, rids)
    return dev_ms, (e2e_ms, e2e_h2d, e2e_d2h), mean_ctx, launches


def prefill_run(engine, vocab, rng, n_prompts=2, prompt_len=1024, reps=5, hold_us=1500):
    """Median time of one step over n_prompts x prompt_len prompt tokens: (device_ms, with_host_ms).
    device_ms: the device's share.  A kernel that only waits (engine.hold) keeps the stream busy while
    the host prepares and queues the step, so the step's copy and kernels run back to back behind it and
    the events bracket them alone.  with_host_ms: the same step timed from the moment the host starts on
    it with an idle device, preparation and launch latency included."""
    import numpy as np

    from sandyrt_b200.engine.step import StepEntry

    prompts = [rng.integers(0, vocab, size=prompt_len, dtype=np.int32) for _ in range(n_prompts)]
    device, with_host = [], []
    for it in range(3 + 2 * reps):
        entries = [StepEntry(f"p{it}-{i}", p, [len(p) - 1]) for i, p in enumerate(prompts)]
        held = it % 2 == 1
        if held:
            engine.hold(hold_us)
        engine.mark(0)
        engine.step(entries)
        engine.mark(1)
        if it >= 3:
            (device if held else with_host).append(engine.elapsed_ms())
        for e in entries:
            engine.release(e.rid)
    engine.check_status()
    return sorted(device)[len(device) // 2], sorted(with_host)[len(with_host) // 2]


def prefill_flops(cfg, n_prompts, prompt_len):
    E, I, L, V = cfg.n_embd, cfg.inner_dim, cfg.n_layer, cfg.vocab_size
    T = n_prompts * prompt_len
    gemm = 2.0 * T * L * (E * 3 * E + E * E + 2 * E * I) + 2.0 * n_prompts * E * V
    attn = L * n_prompts * (2.0 * 2 * E * (prompt_len * (prompt_len + 1) / 2))     # QK^T and PV over the causal half
    return gemm + attn


def roofline_of(llm, model, batch, ctx, ms, peaks):
    weight_bytes = model.weight_bytes()
    kv_bytes = llm.engine.cache.kv_bytes_per_token() * batch * ctx
    gbs = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "of": peaks["source"], "bytes_per_step": weight_bytes + kv_bytes}


def workload(name: str, dtype_name: str, layers: int) -> int:
    """The mixed-batch workloads through LLM.generate.
    medium: 32 requests, prompt lengths uniform in [16, 768], 256 tokens each.
    xl:     64 requests, prompt lengths uniform in [64, 512], 256 tokens each, 16-token pages."""
    import numpy as np

    from sandyrt_b200.engine.llm import LLM

    raw = load_model_config(name)
    n_req, lo, hi = (32, 16, 768) if name == "medium" else (64, 64, 512)
    model, cfg = make_model(raw, layers or raw["n_layer"], dtype_name)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).tolist() for n in rng.integers(lo, hi + 1, size=n_req)]
    llm = LLM(model, dtype=dtype_name, cache_tokens=n_req * 1024, page_size=16, max_live=n_req, max_step_tokens=4096,
              prefill_chunk_tokens=2048)
    llm.generate([p[:32] for p in prompts[:4]], max_tokens=24)              # warm-up: kernels built, graphs recorded
    t0 = time.perf_counter()
    results = llm.generate(prompts, max_tokens=256)
    llm.engine.synchronize()
    wall = time.perf_counter() - t0
    out_tokens = sum(r.completion_tokens for r in results)
    print(json.dumps({
        "workload": name, "dtype": dtype_name, "requests": n_req, "prompt_tokens": sum(len(p) for p in prompts),
        "generated_tokens": out_tokens, "wall_s": wall, "tokens_per_s": out_tokens / wall,
        "total_tokens_per_s": (out_tokens + sum(len(p) for p in prompts)) / wall,
        "preemptions": llm.scheduler.stats["preemptions"], "steps": llm.scheduler.stats["steps"],
        "pages_high_water": [p.high_water for p in llm.engine.cache.alloc.pools], "page_size": 16,
        "n_layer": cfg.n_layer, "n_layer_full": raw["n_layer"], "n_embd": cfg.n_embd, "weights": "random seed 0"}))
    return 0


def attribute(dtype_name: str, layers: int, batch: int, prompts: str = "2x1024", size: str = "small") -> int:
    """What each family of launches costs INSIDE a step: the step is timed whole and again with the
    family left out (its results are garbage then; only the time is read), and the difference is the
    family's share with all overlap between neighbouring kernels as it is in the real step.  A decode
    step of `batch` requests at the bench's context and a prompt step of `prompts` (requests x tokens;
    2 x 1,024 unless --attribute-prompts says otherwise)."""
    import numpy as np

    from sandyrt_b200 import core
    from sandyrt_b200.engine.llm import LLM

    raw = load_model_config(size)
    from sandyrt_b200.config.gpt2 import GPT2Config
    cfg = GPT2Config.from_dict(raw)
    E, I, V = cfg.n_embd, cfg.inner_dim, cfg.vocab_size
    n_prompts, prompt_len = (int(v) for v in prompts.lower().split("x"))
    cases = [("nothing", []), ("layernorm (own launches)", ["layernorm"]), ("attention", ["attention"]),
             (f"q/k/v projection {3 * E}x{E}", [f"product {3 * E}x{E}"]), (f"out-projection {E}x{E}", [f"product {E}x{E}"]),
             (f"up-projection {I}x{E}", [f"product {I}x{E}"]), (f"down-projection {E}x{I}", [f"product {E}x{I}"]),
             (f"vocabulary {V}x{E}", [f"product {V}x{E}"]),
             ("all of these", ["layernorm", "attention", "product"])]
    rows = []
    for name, families in cases:
        model, cfg = make_model(raw, layers or raw["n_layer"], dtype_name)     # an LLM takes its model over
        core.call("global", None, "leave_out", families=families)
        try:
            rng = np.random.default_rng(0)
            llm = LLM(model, cache_tokens=64 * 1024 + 4096, max_live=64, max_step_tokens=4096, prefill_chunk_tokens=2048)
            d_ms, _, ctx, launches = decode_run(llm, batch, 128, 24, 3, rng, V, want_e2e=False)
            p_ms, _ = prefill_run(llm.engine, V, rng, n_prompts=n_prompts, prompt_len=prompt_len, reps=3)
        finally:
            core.call("global", None, "leave_out", families=[])
        rows.append((name, d_ms * 1e3, launches, p_ms * 1e3))
        del llm, model
    d0, p0 = rows[0][1], rows[0][3]
    print(f"{dtype_name}, {cfg.n_layer} layers; decode step of {batch} requests at context ~{ctx:.0f}, prompt step of {n_prompts} x {prompt_len} tokens")
    print(f"  {'left out':32s} {'decode us':>10s} {'saves':>8s} {'per layer':>10s} {'launches':>9s} {'prompt us':>10s} {'saves':>8s} {'per layer':>10s}")
    for name, d, launches, p in rows:
        print(f"  {name:32s} {d:10.1f} {d0 - d:8.1f} {(d0 - d) / cfg.n_layer:10.2f} {launches:9d} {p:10.1f} {p0 - p:8.1f} {(p0 - p) / cfg.n_layer:10.2f}")
    return 0


def profile_kernels(dtype_name: str, layers: int, batch: int, size: str = "small") -> int:
    """Device time per kernel class of one decode step and one 2,048-token prompt step (eager
    launches with a pair of CUDA events around each, so launch gaps are not in the figures)."""
    import numpy as np

    from sandyrt_b200 import core
    from sandyrt_b200.engine.step import Engine, StepEntry

    raw = load_model_config(size)
    model, cfg = make_model(raw, layers or raw["n_layer"], dtype_name)
    engine = Engine(model, max_tokens=batch * 512 + 4096, max_requests=max(batch, 2), max_step_tokens=4096,
                    use_cuda_graphs=False)
    rng = np.random.default_rng(0)
    ids = lambda n: rng.integers(0, cfg.vocab_size, size=n).tolist()
    for i in range(batch):
        engine.step([StepEntry(i, ids(300), [])])
    decode = lambda: engine.step([StepEntry(i, ids(1), [0]) for i in range(batch)])

    def prompt(k):
        for i in range(batch):
            if i in engine.cache.alloc:
                engine.release(i)                         # the prompt step's two requests need slots
        engine.step([StepEntry(f"p{k}a", ids(1024), [1023]), StepEntry(f"p{k}b", ids(1024), [1023])])
        engine.release(f"p{k}a")
        engine.release(f"p{k}b")
    for what, fn, reps in (("decode step, batch %d at context ~300" % batch, lambda k: decode(), 5),
                           ("prompt step, 2 x 1,024 tokens", prompt, 3)):
        fn(-1)                                            # untimed: kernels loaded, products tuned
        core.call("global", None, "profile_kernels", enable=True)
        for k in range(reps):
            fn(k)
        table = core.call("global", None, "profile_kernels", enable=False)
        total = sum(r["us"] for r in table) / reps
        print(f"{what} ({dtype_name}, {cfg.n_layer} layers): {total:.1f} us in kernels per step")
        print("  class                     calls      us   share    GB/s  TFLOP/s")
        for r in sorted(table, key=lambda r: -r["us"]):
            us = r["us"] / reps
            gbs = r["bytes"] / reps / us / 1e3 if us else 0.0
            tf = r["flops"] / reps / us / 1e6 if us else 0.0
            print(f"  {r['class']:24s} {r['calls'] // reps:6d} {us:7.1f} {100 * us / total:6.1f}% {gbs:7.0f} {tf:8.1f}")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="dtype of --workload / --profile-kernels")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points and the float32 block")
    ap.add_argument("--workload", choices=["medium", "xl"], help="run a mixed-batch workload through LLM.generate instead")
    ap.add_argument("--profile-kernels", action="store_true", help="print device time per kernel class instead")
    ap.add_argument("--under-profiler", action="store_true",
                    help="skip the check of the device time against the wall clock (a profiler serialises the launches)")
    ap.add_argument("--attribute", action="store_true", help="print what each family of launches costs inside a step instead")
    ap.add_argument("--size", default="small", choices=["small", "medium", "xl"], help="model size of --attribute / --profile-kernels")
    ap.add_argument("--attribute-prompts", default="2x1024", help="the prompt step of --attribute: requests x tokens")
    ap.add_argument("--micro", nargs=argparse.REMAINDER, help="run a kernel micro-benchmark (see sandyrt_b200/csrc/microbench.py)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    if args.micro is not None:
        from sandyrt_b200.csrc import microbench
        return microbench.main(args.micro)
    if args.workload:
        return workload(args.workload, args.dtype, args.layers)
    if args.profile_kernels:
        return profile_kernels(args.dtype, args.layers, args.batch, args.size)
    if args.attribute:
        return attribute(args.dtype, args.layers, args.batch, args.attribute_prompts, args.size)
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np

    from sandyrt_b200.engine.llm import LLM

    peaks = load_peaks()
    raw = load_model_config("small")
    model, cfg = make_model(raw, args.layers or raw["n_layer"], "bfloat16")
    vocab = cfg.vocab_size
    rng = np.random.default_rng(0)
    llm = LLM(model, cache_tokens=64 * 1024 + 4096, max_live=64, max_step_tokens=4096, prefill_chunk_tokens=2048)
    engine = llm.engine

    clocks = ClockSampler()
    clocks.start()

    # ---- decode at the headline batch ------------------------------------------------------------
    dev_ms, (wall_ms, e2e_h2d, e2e_d2h), mean_ctx, launches_per_step = decode_run(
        llm, args.batch, args.prompt_len, args.steps, args.warmup, rng, vocab)
    if dev_ms > wall_ms * 1.05 and not args.under_profiler:
        raise RuntimeError(f"device time {dev_ms:.4f} ms a step exceeds the wall-clock {wall_ms:.4f} ms of the same work")
    value = args.batch / (dev_ms / 1e3)
    e2e_value = args.batch / (wall_ms / 1e3)
    roofline = roofline_of(llm, model, args.batch, mean_ctx, dev_ms, peaks)

    # ---- prefill of 2,048 tokens: 2 prompts x 1,024 in one step ----------------------------------
    pf_ms, pf_host_ms = prefill_run(engine, vocab, rng)
    pf_frac = prefill_flops(cfg, 2, 1024) / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)

    points, fp32 = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            d_ms, _, ctx, _ = decode_run(llm, b, args.prompt_len, min(args.steps, 128), args.warmup, rng, vocab, want_e2e=False)
            points[f"decode_b{b}"] = {"value": b / (d_ms / 1e3), "ms_per_step": d_ms, "mean_context": round(ctx, 1),
                                      "roofline_frac": roofline_of(llm, model, b, ctx, d_ms, peaks)["frac"]}
        # the float32 path (FFMA products, float cache): the same model in float32
        model32, _ = make_model(raw, args.layers or raw["n_layer"], "float32")
        llm32 = LLM(model32, dtype="float32", cache_tokens=16 * 1024 + 4096, max_live=16, max_step_tokens=4096,
                    prefill_chunk_tokens=2048)
        for b in (1, 8):
            d_ms, _, ctx, _ = decode_run(llm32, b, args.prompt_len, min(args.steps, 32), 3, rng, vocab, want_e2e=False)
            fp32[f"decode_b{b}"] = {"value": b / (d_ms / 1e3), "ms_per_step": d_ms, "mean_context": round(ctx, 1)}
        p32, _ = prefill_run(llm32.engine, vocab, rng, reps=2)
        fp32["prefill"] = {"value": 2048 / (p32 / 1e3), "tokens": 2048, "ms": p32}

    clock_info = clocks.stop()
    out = {
        "metric": "decode tok/s at batch 8 (GPT-2 small)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "gpt2-small", "n_layer": cfg.n_layer, "n_layer_full": raw["n_layer"], "n_embd": cfg.n_embd,
                   "n_head": cfg.n_head, "head_dim": cfg.head_dim, "n_inner": cfg.inner_dim, "vocab_size": vocab,
                   "n_positions": cfg.n_positions, "global_batch": args.batch, "seq_len": cfg.n_positions,
                   "prompt_len": args.prompt_len, "mean_context": round(mean_ctx, 1), "page_size": 16,
                   "parallelism": "single-gpu", "weights": "random seed 0", "host": "C++ core (libsandy_core)",
                   "l2": "inputs larger than L2 (weights %.0f MB)" % (model.weight_bytes() / 1e6)},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": wall_ms,
                "h2d_bytes_per_step": round(e2e_h2d, 1), "d2h_bytes_per_step": round(e2e_d2h, 1),
                "steps_per_burst": 8, "bursts_queued_ahead": True},
        "gpu_launches": launches_per_step * args.steps, "launches_per_step": launches_per_step,
        "prefill": {"value": 2048 / (pf_ms / 1e3), "tokens": 2048, "ms": pf_ms, "ms_with_host": pf_host_ms, "frac": pf_frac,
                    "peak": f"{peaks['bf16_tflops']} TFLOP/s bf16 of {peaks['source']}"},
        "roofline": roofline,
        "points": points,
        "fp32": fp32,
        "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
