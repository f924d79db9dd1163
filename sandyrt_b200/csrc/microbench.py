"""Kernel micro-benchmarks: one kernel alone, inside a CUDA graph, on inputs larger than L2.

    python -m sandyrt_b200.csrc.microbench decode-attention [--heads 12] [--head-dim 64] [--page-size 16]
    python -m sandyrt_b200.csrc.microbench gemm [--rows 2048] [--width 768] [--inner 3072] [--layers 48] [--k-sweep]
    python -m sandyrt_b200.csrc.microbench prefill-attention [--heads 12] [--page-size 16] [--shape 2x1024+0 ...]

decode-attention: the register kernel and the bulk-copy kernel of single-token attention on
several (tokens, context) shapes.  Each timing replays a graph of one launch per distinct cache
(enough caches to exceed L2), so neither the host's launch cost nor a warm L2 is in the number;
bytes are the keys and values a launch must read.

prefill-attention: the mma.sync kernel and the tcgen05 kernel of prompt attention (heads of 64)
on shapes given as REQUESTSxNEW+CACHED, with the requests' pages one after another in the cache
and scattered; FLOP are those of the causal part (4 * head * keys seen, per query and head).
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import ops


def _time_graph(fn, layers: int, reps: int = 3) -> float:
    """Microseconds per call of fn(l), l = 0..layers-1, replayed from a CUDA graph."""
    for l in range(layers):
        fn(l)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fn(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for l in range(layers):
                fn(l)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * layers)


def decode_attention(a) -> int:
    dev = torch.device("cuda:0")
    H, D, PS = a.heads, a.head_dim, a.page_size
    print("tokens context  kernel    splits       us     GB/s")
    shapes = [tuple(int(v) for v in sh.split("x")) for sh in a.shape]
    for T, ctx in shapes:
        blocks = -(-ctx // PS)
        pages = T * blocks
        bytes_per_launch = T * ctx * H * D * 2 * 2
        layers = min(48, max(2, int(400e6 // bytes_per_launch) + 1))
        arena = torch.randn(layers, pages, 2, H, PS, D, device=dev, dtype=torch.bfloat16)
        table = torch.randperm(pages, device=dev).to(torch.int32).view(T, blocks).contiguous()
        q = torch.randn(T, H * D, device=dev, dtype=torch.bfloat16)
        seq = torch.arange(T, device=dev, dtype=torch.int32)
        pos = torch.full((T,), ctx - 1, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        splits = min(ops.decode_splits(T, H, blocks * PS), ops.CLUSTER_MAX_SPLITS)
        kernels = [("register", dict(bulk=False)), ("bulk", dict(bulk=True))]
        if D == 64:
            kernels.append(("mma.sync", dict(mma=True)))
        for name, which in kernels:
            def go(l, which=which):
                ops.decode_attention(q, arena[l, :, 0], arena[l, :, 1], table, seq, pos, out, n_heads=H,
                                     scale=D ** -0.5, num_splits=splits, cluster=True, **which)
            us = _time_graph(go, layers)
            print(f"{T:6d} {ctx:7d}  {name:8s} {splits:6d} {us:8.2f} {bytes_per_launch / us / 1e3:8.0f}", flush=True)
        ops.check_kernel_status(dev)
        del arena
    return 0


def gemm(a) -> int:
    """The tcgen05 product at the shapes of a prompt step, every tile choice; activations and
    weights of --layers distinct layers (48 by default: 170 to 230 MB of weights per shape, more
    than L2 holds, so the weights come from memory as they do in a model)."""
    dev = torch.device("cuda:0")
    M = a.rows
    shapes = [("q/k/v", 3 * a.width, a.width, None, False), ("out-projection", a.width, a.width, None, True),
              ("up-projection", a.inner, a.width, "gelu_new", False), ("down-projection", a.width, a.inner, None, True)]
    print(f"rows {M}; us per launch (TFLOP/s) by tile width; negative: one tile per CTA; 2000+: two CTAs a tile")
    layers = a.layers
    for name, N, K, act, res in shapes:
        # inputs are a kernel's output in a model and sit in L2; four of them take turns here
        x4 = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(4)]
        xs = [x4[l % 4] for l in range(layers)]
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(layers)]
        bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
        # the residual products add into the float32 stream in place, as the blocks do
        out = torch.zeros(M, N, device=dev, dtype=torch.float32 if res else torch.bfloat16)
        resid = out if res else None
        line = f"{name:16s} {M}x{N}x{K}:"
        for tile in ops.GEMM_VARIANTS:
            def go(l, tile=tile):
                ops.gemm_tc(xs[l], ws[l], bias, out, act=act, residual=resid, tile_n=tile)
            us = _time_graph(go, layers)
            line += f"  {tile:5d}: {us:6.1f} ({2.0 * M * N * K / us / 1e6:5.0f})"
        if M <= ops.SKINNY_MAX_ROWS:
            def go_skinny(l):
                ops.gemm_skinny(xs[l], ws[l], bias, out, act=act, residual=resid)
            line += f"  skinny: {_time_graph(go_skinny, layers):6.1f}"

            def go_small(l):
                ops.gemm_small(xs[l], ws[l], bias, out, act=act, residual=resid)
            line += f"  small ({ops.gemm_small_splits(N, K)} splits): {_time_graph(go_small, layers):6.1f}"
        # the library's product with its bias alone (no activation, no residual, bfloat16 out): the yardstick
        lib_out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

        def go_lib(l):
            torch.addmm(bias, xs[l], ws[l].t(), out=lib_out)
        us = _time_graph(go_lib, layers)
        line += f"  cuBLAS: {us:6.1f} ({2.0 * M * N * K / us / 1e6:5.0f})"
        print(line, flush=True)
        ops.check_kernel_status(dev)
    if a.k_sweep:
        # the q/k/v output size at several K, no bias: what does not move with K is launch,
        # set-up and write-back; the slope is the main loop's rate
        N = 3 * a.width
        print(f"K sweep at {M}x{N}, no bias, bfloat16 out: us (TFLOP/s)")
        for K in (64, 256, 768, 1536, 3072):
            x4 = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(4)]
            xs = [x4[l % 4] for l in range(layers)]
            ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(layers)]
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            line = f"K {K:5d}:"
            for tile in (128, ops.PAIR_TILE + 256):
                def go(l, tile=tile):
                    ops.gemm_tc(xs[l], ws[l], None, out, tile_n=tile)
                us = _time_graph(go, layers)
                line += f"  {tile:5d}: {us:6.1f} ({2.0 * M * N * K / us / 1e6:5.0f})"
            print(line, flush=True)
    return 0


def prefill_attention(a) -> int:
    import math

    dev = "cuda:0"
    H, D, ps = a.heads, 64, a.page_size
    print(f"prefill attention, {H} heads of {D}, pages of {ps}; us per launch and TFLOP/s of the causal part")
    for shape in a.shape:
        reqs, rest = shape.split("x")
        new, cached = rest.split("+")
        n_seqs, q_len, before = int(reqs), int(new), int(cached)
        L = before + q_len
        nb = -(-L // ps)
        num_pages = n_seqs * nb + 1
        g = torch.Generator(device=dev).manual_seed(0)
        arena = torch.randn(num_pages, 2, H, ps, D, device=dev, generator=g).to(torch.bfloat16)
        kc, vc = arena[:, 0], arena[:, 1]
        T = n_seqs * q_len
        q = torch.randn(T, H * D, device=dev, generator=g).to(torch.bfloat16)
        q_start = torch.arange(0, T + 1, q_len, dtype=torch.int32, device=dev)
        kv_before = torch.full((n_seqs,), before, dtype=torch.int32, device=dev)
        flops = 4.0 * n_seqs * H * D * sum(before + i + 1 for i in range(q_len))
        tables = {"runs": torch.arange(n_seqs * nb, device=dev, dtype=torch.int32).view(n_seqs, nb).contiguous(),
                  "scattered": torch.randperm(num_pages - 1, device=dev, generator=g).to(torch.int32)[:n_seqs * nb]
                  .view(n_seqs, nb).contiguous()}
        outs = {}
        for pages, table in tables.items():
            for name, tc in (("mma.sync", False), ("tcgen05", True)):
                out = torch.zeros_like(q)

                def go(l, table=table, tc=tc, out=out):
                    ops.prefill_attention(q, kc, vc, table, q_start, kv_before, out, n_heads=H, max_q_len=q_len,
                                          scale=1 / math.sqrt(D), tc=tc)
                us = _time_graph(go, a.launches)
                ops.check_kernel_status(dev)
                outs[name] = out.float()
                print(f"  {shape:>12} pages {pages:>9} {name:>8}: {us:7.1f} us  {flops / us / 1e6:6.0f} TFLOP/s", flush=True)
            print(f"  {'':>12} largest difference between the two kernels: "
                  f"{(outs['tcgen05'] - outs['mma.sync']).abs().max().item():.4f}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sandyrt_b200.csrc.microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("decode-attention")
    d.add_argument("--heads", type=int, default=12)
    d.add_argument("--head-dim", type=int, default=64)
    d.add_argument("--page-size", type=int, default=16)
    d.add_argument("--shape", nargs="+", default=["64x384", "64x1024", "256x384", "8x384", "8x1024", "1x1024"],
                   help="tokens x context")
    d.set_defaults(fn=decode_attention)
    g = sub.add_parser("gemm")
    g.add_argument("--rows", type=int, default=2048)
    g.add_argument("--width", type=int, default=768)
    g.add_argument("--inner", type=int, default=3072)
    g.add_argument("--k-sweep", action="store_true", help="also time the q/k/v output size at several K")
    g.add_argument("--layers", type=int, default=48, help="distinct weights and inputs per shape")
    g.set_defaults(fn=gemm)
    pa = sub.add_parser("prefill-attention")
    pa.add_argument("--heads", type=int, default=12)
    pa.add_argument("--page-size", type=int, default=16)
    pa.add_argument("--launches", type=int, default=20, help="launches per timed graph")
    pa.add_argument("--shape", nargs="+", default=["2x1024+0", "8x256+0", "4x512+512", "16x128+0", "2x2048+0", "1x8192+0"],
                    help="REQUESTSxNEW+CACHED")
    pa.set_defaults(fn=prefill_attention)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
