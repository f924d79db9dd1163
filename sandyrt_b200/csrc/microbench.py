"""Kernel micro-benchmarks: one kernel alone, inside a CUDA graph, on inputs larger than L2.

    python -m sandyrt_b200.csrc.microbench decode-attention [--heads 12] [--head-dim 64] [--page-size 16]
    python -m sandyrt_b200.csrc.microbench gemm [--rows 2048] [--width 768] [--inner 3072] [--k-sweep]

decode-attention: the register kernel and the bulk-copy kernel of single-token attention on
several (tokens, context) shapes.  Each timing replays a graph of one launch per distinct cache
(enough caches to exceed L2), so neither the host's launch cost nor a warm L2 is in the number;
bytes are the keys and values a launch must read.
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
    for T, ctx in ((64, 384), (64, 1024), (256, 384), (8, 384), (8, 1024), (1, 1024)):
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
        for bulk in (False, True):
            def go(l, bulk=bulk):
                ops.decode_attention(q, arena[l, :, 0], arena[l, :, 1], table, seq, pos, out, n_heads=H,
                                     scale=D ** -0.5, num_splits=splits, cluster=True, bulk=bulk)
            us = _time_graph(go, layers)
            print(f"{T:6d} {ctx:7d}  {'bulk' if bulk else 'register':8s} {splits:6d} {us:8.2f} {bytes_per_launch / us / 1e3:8.0f}",
                  flush=True)
        ops.check_kernel_status(dev)
        del arena
    return 0


def gemm(a) -> int:
    """The tcgen05 product at the shapes of a prompt step, every tile choice; activations and
    weights of `layers` distinct layers so that the operands do not sit in L2 between launches."""
    dev = torch.device("cuda:0")
    M = a.rows
    shapes = [("q/k/v", 3 * a.width, a.width, None, False), ("out-projection", a.width, a.width, None, True),
              ("up-projection", a.inner, a.width, "gelu_new", False), ("down-projection", a.width, a.inner, None, True)]
    print(f"rows {M}; us per launch (TFLOP/s) by tile width; negative: one tile per CTA; 2000+: two CTAs a tile")
    layers = 12
    for name, N, K, act, res in shapes:
        xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(layers)]
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(layers)]
        bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.float32 if res else torch.bfloat16)
        resid = torch.randn(M, N, device=dev, dtype=torch.float32) if res else None
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
        print(line, flush=True)
        ops.check_kernel_status(dev)
    if a.k_sweep:
        # the q/k/v output size at several K, no bias: what does not move with K is launch,
        # set-up and write-back; the slope is the main loop's rate
        N = 3 * a.width
        print(f"K sweep at {M}x{N}, no bias, bfloat16 out: us (TFLOP/s)")
        for K in (64, 256, 768, 1536, 3072):
            xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) for _ in range(layers)]
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sandyrt_b200.csrc.microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("decode-attention")
    d.add_argument("--heads", type=int, default=12)
    d.add_argument("--head-dim", type=int, default=64)
    d.add_argument("--page-size", type=int, default=16)
    d.set_defaults(fn=decode_attention)
    g = sub.add_parser("gemm")
    g.add_argument("--rows", type=int, default=2048)
    g.add_argument("--width", type=int, default=768)
    g.add_argument("--inner", type=int, default=3072)
    g.add_argument("--k-sweep", action="store_true", help="also time the q/k/v output size at several K")
    g.set_defaults(fn=gemm)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
