"""Decode programs: a step's kernels described as data and run by one resident kernel.

While a `Recorder` is installed (`recording(...)`), the functions of `ops` that a decode
step uses do not launch anything: they append a record of what they would have launched.
The finished list is a `Program`; `Program.run()` hands it to the interpreter kernel
(decode_program.cu), which walks it with a grid-wide barrier between operations.  An
operation the interpreter does not know, or sizes it does not take, raise `NotRecordable`
during recording; the caller then runs the step through the ordinary kernels instead.

The records hold raw device addresses, so a program is only valid while the tensors it names
stay where they are: the engine keys programs like its CUDA graphs (step shape, staging
buffer, workspace version) and the program itself keeps a reference to every tensor.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Dict, List, Optional

import torch

from .build import load_library

OP_EMBED, OP_NORM, OP_GEMM, OP_ATTN = 0, 1, 2, 3


class NotRecordable(Exception):
    """The step uses an operation or a size the program interpreter does not take."""


class Op(ctypes.Structure):
    """Mirror of `struct Op` in decode_program.cu.  Fields by kind:

    EMBED  M rows, N width, ldc; ids, positions, w (token table), wpe (position table or null),
           vocab, n_pos, out (float), status
    NORM   M rows, K width, ldx, ldc; x (float), rows (gather or null), gamma, beta, eps, out (bfloat16)
    GEMM   M, N, K, lda, ldw, ldr, ldc, act, out_dtype; a (bfloat16) or x/ldx/gamma/beta/eps (fused
           norm), w [N, K], bias, residual (float), out; with k_cache: v_cache, page_stride,
           block_table, max_blocks, token_seq, positions, q_cols, kv_cols, head_dim, page_size,
           num_pages; status
    ATTN   M tokens, a = q with ld_q, out with ldc, k_cache, v_cache, page_stride, block_table,
           max_blocks, token_seq, positions, n_heads, n_kv_heads, head_dim, page_size, num_pages,
           window, scale, num_splits, partial, counters, status
    table_slot (GEMM with k_cache, ATTN): which of the program's cached block tables the record's
    block_table is, or -1 to read positions, token_seq and block_table from global memory.
    """
    _fields_ = [(n, ctypes.c_int) for n in (
        "kind", "M", "N", "K", "lda", "ldw", "ldr", "ldc", "act", "out_dtype", "ldx", "max_blocks",
        "q_cols", "kv_cols", "head_dim", "page_size", "num_pages", "n_heads", "n_kv_heads", "window",
        "num_splits", "vocab", "n_pos", "ld_q", "table_slot", "flags")] + [
        ("eps", ctypes.c_float), ("scale", ctypes.c_float), ("page_stride", ctypes.c_longlong)] + [
        (n, ctypes.c_void_p) for n in (
            "a", "x", "gamma", "beta", "w", "bias", "residual", "out", "k_cache", "v_cache", "block_table",
            "token_seq", "positions", "rows", "ids", "wpe", "partial", "counters", "status", "reserved")]


class StepArrays(ctypes.Structure):
    """Mirror of `struct StepArrays`: the step's index arrays, cached in shared memory by every block."""
    _fields_ = [("positions", ctypes.c_void_p), ("token_seq", ctypes.c_void_p),
                ("tables", ctypes.c_void_p * 4), ("max_blocks", ctypes.c_int * 4),
                ("n_tokens", ctypes.c_int), ("n_seqs", ctypes.c_int), ("n_tables", ctypes.c_int),
                ("pad", ctypes.c_int)]


_limits: Optional[Dict[str, int]] = None
_sync: Dict[int, torch.Tensor] = {}


def limits() -> Dict[str, int]:
    global _limits
    if _limits is None:
        lib = load_library("decode_program")
        names = ("max_rows", "a_bytes", "op_bytes", "sync_bytes", "row_pad", "max_norm_width", "table_ints",
                 "max_tables", "arrays_bytes")
        vals = [ctypes.c_int(0) for _ in names]
        lib.sandy_decode_program_limits(*[ctypes.byref(v) for v in vals])
        _limits = {n: v.value for n, v in zip(names, vals)}
        if _limits["op_bytes"] != ctypes.sizeof(Op) or _limits["arrays_bytes"] != ctypes.sizeof(StepArrays) \
                or _limits["max_tables"] != 4:
            raise RuntimeError(f"decode program: the records are {ctypes.sizeof(Op)} and {ctypes.sizeof(StepArrays)} "
                               f"bytes here, {_limits['op_bytes']} and {_limits['arrays_bytes']} in the kernel")
        grid = ctypes.c_int(0)
        code = lib.sandy_decode_program_grid(ctypes.byref(grid))
        if code != 0:
            raise RuntimeError(f"decode program: cannot read the device's SM count (CUDA error {code})")
        _limits["grid"] = grid.value
    return _limits


def _sync_buffer(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    t = _sync.get(key)
    if t is None:
        t = torch.zeros(max(3, limits()["sync_bytes"] // 8), dtype=torch.int64, device=device)
        _sync[key] = t
    return t


def reset_sync() -> None:
    """After a launch that gave up on a wait the barrier counter is meaningless: start over."""
    for t in _sync.values():
        t.zero_()


class Program:
    def __init__(self, ops: List[Op], keep: List[torch.Tensor], device, status: torch.Tensor,
                 arrays: StepArrays):
        self.n_ops = len(ops)
        self.arrays = arrays
        raw = b"".join(bytes(o) for o in ops)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.records = host.to(device)
        self.keep = keep
        self.device = device
        self.status = status
        self.sync = _sync_buffer(device)
        self.kinds = [o.kind for o in ops]

    def run(self, timeline: Optional[torch.Tensor] = None) -> None:
        """One launch on torch's current stream.  timeline: int64 [3 * n_ops + 1] on the device, filled
        with block 0's nanosecond clock: [0] at the start, then for each operation two marks inside
        it (activations staged or first keys merged; work done) and the time after its barrier."""
        from . import ops as _ops
        if timeline is not None and (timeline.dtype != torch.int64 or timeline.numel() < 3 * self.n_ops + 1
                                     or not timeline.is_cuda):
            raise ValueError("timeline must be a CUDA int64 tensor of 3 * n_ops + 1 elements")
        lib = load_library("decode_program")
        code = lib.sandy_decode_program_run(ctypes.c_void_p(self.records.data_ptr()), ctypes.c_int(self.n_ops),
                                            ctypes.c_void_p(self.sync.data_ptr()),
                                            ctypes.c_void_p(self.status.data_ptr()),
                                            ctypes.c_void_p(0 if timeline is None else timeline.data_ptr()),
                                            ctypes.byref(self.arrays), _ops._stream())
        _ops._check(code, f"decode_program({self.n_ops} operations)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Recorder:
    """Collects the records of one step.  The `ops` functions call these methods after their own
    argument checks, with the tensors they would have passed to their kernels."""

    def __init__(self, device, status: torch.Tensor):
        self.device = device
        self.status = status            # where waits that ran out and missing pages are reported
        self.ops: List[Op] = []
        self.keep: List[torch.Tensor] = []
        self.lim = limits()
        self._partial: Optional[torch.Tensor] = None
        self._counters: Optional[torch.Tensor] = None
        # the step's index arrays, as the first record that names them gives them
        self._positions: Optional[torch.Tensor] = None
        self._token_seq: Optional[torch.Tensor] = None
        self._tables: List[torch.Tensor] = []
        self._uncached = False

    def _table_slot(self, block_table, token_seq, positions) -> int:
        """Which cached block table this is (-1: the record reads the arrays from global memory)."""
        if self._positions is None:
            self._positions, self._token_seq = positions, token_seq
        if positions.data_ptr() != self._positions.data_ptr() or token_seq.data_ptr() != self._token_seq.data_ptr() \
                or positions.numel() != self._positions.numel():
            self._uncached = True
            return -1
        for i, t in enumerate(self._tables):
            if t.data_ptr() == block_table.data_ptr() and t.shape == block_table.shape:
                return i
        if len(self._tables) >= self.lim["max_tables"]:
            return -1
        if self._tables and block_table.shape[0] != self._tables[0].shape[0]:
            return -1
        self._tables.append(block_table)
        return len(self._tables) - 1

    def _hold(self, *tensors) -> None:
        self.keep.extend(t for t in tensors if t is not None)

    def _rows(self, M: int) -> None:
        if M > self.lim["max_rows"]:
            raise NotRecordable(f"{M} rows (the interpreter takes {self.lim['max_rows']})")

    # ---- one method per operation ---------------------------------------------------------
    def embed(self, ids, positions, wte, wpe, out, status) -> None:
        M, width = out.shape
        self._rows(M)
        if wte.dtype != torch.bfloat16 or out.dtype != torch.float32:
            raise NotRecordable("embedding: bfloat16 table into a float32 stream only")
        op = Op(kind=OP_EMBED, M=M, N=width, ldc=out.stride(0), vocab=wte.shape[0],
                n_pos=0 if wpe is None else wpe.shape[0])
        op.ids, op.positions, op.w, op.wpe, op.out = _ptr(ids), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out)
        op.status = _ptr(status)
        self._hold(ids, positions, wte, wpe, out, status)
        self.ops.append(op)

    def norm(self, x, gamma, beta, eps, out, rows) -> None:
        M, K = out.shape
        self._rows(M)
        if x.dtype != torch.float32 or out.dtype != torch.bfloat16 or gamma.dtype != torch.bfloat16 \
                or K > self.lim["max_norm_width"] or K % 4 or x.stride(0) % 4 or x.data_ptr() % 16 \
                or out.stride(0) % 4 or out.data_ptr() % 8 or gamma.data_ptr() % 8 \
                or (beta is not None and (beta.dtype != torch.bfloat16 or beta.data_ptr() % 8)):
            raise NotRecordable(f"norm of width {K}, {x.dtype} -> {out.dtype}")
        op = Op(kind=OP_NORM, M=M, K=K, ldx=x.stride(0), ldc=out.stride(0), eps=eps)
        op.x, op.gamma, op.beta, op.out, op.rows = _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(rows)
        self._hold(x, gamma, beta, out, rows)
        self.ops.append(op)

    def gemm(self, a, x, gamma, beta, eps, w, bias, residual, out, act_code: int, out_dtype: int, kv) -> None:
        M, N = out.shape
        K = w.shape[1]
        self._rows(M)
        if M * (K + self.lim["row_pad"]) * 2 > self.lim["a_bytes"]:
            raise NotRecordable(f"{M} rows of {K} do not fit the interpreter's shared memory")
        if x is not None and (K > self.lim["max_norm_width"] or K % 8 or gamma.data_ptr() % 16
                              or (beta is not None and beta.data_ptr() % 16)):
            raise NotRecordable(f"fused norm of width {K}")
        if bias is not None and bias.data_ptr() % 16:
            raise NotRecordable("a bias that does not start on a 16-byte boundary")
        op = Op(kind=OP_GEMM, M=M, N=N, K=K, lda=0 if a is None else a.stride(0), ldw=w.stride(0),
                ldr=0 if residual is None else residual.stride(0), ldc=out.stride(0), act=act_code,
                out_dtype=out_dtype, ldx=0 if x is None else x.stride(0), eps=eps)
        op.a, op.x, op.gamma, op.beta = _ptr(a), _ptr(x), _ptr(gamma), _ptr(beta)
        op.w, op.bias, op.residual, op.out = _ptr(w), _ptr(bias), _ptr(residual), _ptr(out)
        op.status = _ptr(self.status)
        self._hold(a, x, gamma, beta, w, bias, residual, out)
        if kv is not None:
            kc, vc, table, tseq, tpos, page_stride, q_cols, kv_cols, head_dim, page_size, num_pages = kv
            op.k_cache, op.v_cache, op.block_table = _ptr(kc), _ptr(vc), _ptr(table)
            op.token_seq, op.positions = _ptr(tseq), _ptr(tpos)
            op.page_stride, op.max_blocks = page_stride, table.shape[1]
            op.q_cols, op.kv_cols, op.head_dim, op.page_size, op.num_pages = q_cols, kv_cols, head_dim, page_size, num_pages
            op.table_slot = self._table_slot(table, tseq, tpos)
            self._hold(kc, vc, table, tseq, tpos)
        self.ops.append(op)

    def attention(self, q, k_cache, v_cache, page_stride, num_pages, block_table, token_seq, positions, out, *,
                  n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, scale: float, window: int) -> None:
        M = q.shape[0]
        self._rows(M)
        if q.dtype != torch.bfloat16 or head_dim not in (16, 32, 64, 128, 256) or q.stride(0) % 8 \
                or q.data_ptr() % 16 or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16 or page_stride % 8:
            raise NotRecordable(f"attention with head size {head_dim} in {q.dtype}")
        grid = self.lim["grid"]
        pairs = M * n_heads
        max_kv = block_table.shape[1] * page_size
        # one unit a block where the pairs allow it (the merge of splits costs two more trips to
        # memory), and no unit under 64 keys
        splits = max(1, min(grid // pairs, -(-max_kv // 64), 32))
        need = pairs * splits * (head_dim + 2)
        if self._partial is None or self._partial.numel() < need:
            self._partial = torch.empty(need, dtype=torch.float32, device=self.device)
        if self._counters is None or self._counters.numel() < pairs:
            self._counters = torch.zeros(pairs, dtype=torch.int32, device=self.device)
        op = Op(kind=OP_ATTN, M=M, ld_q=q.stride(0), ldc=out.stride(0), max_blocks=block_table.shape[1],
                n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=page_size,
                num_pages=num_pages, window=window, num_splits=splits, scale=scale, page_stride=page_stride)
        op.a, op.out, op.k_cache, op.v_cache = _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache)
        op.block_table, op.token_seq, op.positions = _ptr(block_table), _ptr(token_seq), _ptr(positions)
        op.table_slot = self._table_slot(block_table, token_seq, positions)
        op.status = _ptr(self.status)
        self._hold(q, out, k_cache, v_cache, block_table, token_seq, positions)
        self.ops.append(op)

    def finish(self) -> Program:
        # every attention record shares one scratch (they run one after the other); it may have
        # grown while recording, so the addresses go in last
        for op in self.ops:
            if op.kind == OP_ATTN:
                op.partial, op.counters = _ptr(self._partial), _ptr(self._counters)
        self._hold(self._partial, self._counters)
        arrays = StepArrays()
        ints = sum(t.numel() for t in self._tables)
        if self._tables and not self._uncached and ints <= self.lim["table_ints"] \
                and self._positions.numel() <= self.lim["max_rows"]:
            arrays.positions, arrays.token_seq = _ptr(self._positions), _ptr(self._token_seq)
            arrays.n_tokens, arrays.n_seqs = self._positions.numel(), self._tables[0].shape[0]
            arrays.n_tables = len(self._tables)
            for i, t in enumerate(self._tables):
                arrays.tables[i], arrays.max_blocks[i] = _ptr(t), t.shape[1]
        else:
            for op in self.ops:
                op.table_slot = -1
        return Program(self.ops, self.keep, self.device, self.status, arrays)


@contextlib.contextmanager
def recording(device, status: torch.Tensor):
    """Install a Recorder for the `ops` functions called inside the block."""
    from . import ops as _ops
    if _ops._recorder is not None:
        raise RuntimeError("a decode program is already being recorded")
    rec = Recorder(device, status)
    _ops._recorder = rec
    try:
        yield rec
    finally:
        _ops._recorder = None
