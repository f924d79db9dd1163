"""The decode-attention entry point that allocates nothing (sandy_decode_attention_static).

It exists for callers that cannot give the split-KV kernel a scratch buffer because they may
not allocate device memory where they run; its scratch is a fixed 4 MiB array inside the
library.  The test calls it through its exported C symbol, twice in a row with different
inputs (the array keeps the first call's contents: nothing of them may leak into the second
result), and compares each result with the ordinary entry point's, which is given a scratch
tensor.  It also checks that a shape beyond the array's size is refused before anything runs.

The file's name makes pytest collect it last, so a run that stops at the first failure has
run every other test by then.  It passes alone in a fresh process as well as after the others.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, dtype, H, D, page_size, lens):
    """Single-token queries over contexts `lens`, pages handed out in shuffled order."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blocks = [-(-n // page_size) for n in lens]
    num_pages = sum(n_blocks) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(lens), max(n_blocks)), -1, dtype=torch.int32)
    arena = torch.randn(num_pages, 2, H, page_size, D, generator=g).to(dtype)
    for s, nb in enumerate(n_blocks):
        for b in range(nb):
            table[s, b] = perm.pop()
    q = torch.randn(len(lens), H * D, generator=g).to(dtype)
    arena = arena.to(DEV)
    return dict(q=q.to(DEV), kc=arena[:, 0], vc=arena[:, 1], table=table.to(DEV),
                tok_seq=torch.arange(len(lens), dtype=torch.int32, device=DEV),
                tok_pos=torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV))


def _call_static(lib, c, out, H, D, page_size, scale, splits, status):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    kc = c["kc"]
    return lib.sandy_decode_attention_static(
        p(c["q"]), ctypes.c_int(c["q"].stride(0)), p(kc), p(c["vc"]), ctypes.c_longlong(kc.stride(0)),
        p(c["table"]), ctypes.c_int(c["table"].shape[1]), p(c["tok_seq"]), p(c["tok_pos"]), p(out),
        ctypes.c_int(out.stride(0)), ctypes.c_int(c["q"].shape[0]), ctypes.c_int(H), ctypes.c_int(H), ctypes.c_int(D),
        ctypes.c_int(page_size), ctypes.c_float(scale), ctypes.c_int(0), ctypes.c_int(splits),
        ctypes.c_int(kc.shape[0]), ctypes.c_int(1 if c["q"].dtype == torch.bfloat16 else 0), p(status),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from sandyrt_b200.csrc import ops
    from sandyrt_b200.csrc.build import load_library

    lib = load_library("attention_decode")
    lib.sandy_decode_attention_static_strerror.restype = ctypes.c_char_p
    lib.sandy_decode_attention_static_capacity.restype = ctypes.c_longlong
    assert lib.sandy_decode_attention_static_capacity() == 1 << 20
    H, D, page_size, splits = 6, 64, 16, 5
    scale = 1.0 / math.sqrt(D)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # two calls in a row: other inputs, other context lengths, same static array
    for seed, lens in ((1, [700, 3, 129, 64, 257]), (2, [40, 512, 1, 333, 90])):
        c = _case(seed, dtype, H, D, page_size, lens)
        got = torch.full_like(c["q"], float("nan"))
        code = _call_static(lib, c, got, H, D, page_size, scale, splits, status)
        assert code == 0, lib.sandy_decode_attention_static_strerror(code).decode()
        want = torch.full_like(c["q"], float("nan"))
        scratch = torch.empty(len(lens) * H * splits * (D + 2), dtype=torch.float32, device=DEV)
        ops.decode_attention(c["q"], c["kc"], c["vc"], c["table"], c["tok_seq"], c["tok_pos"], want,
                             n_heads=H, scale=scale, num_splits=splits, scratch=scratch)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert not torch.isnan(got).any()
        # both entry points run the same kernels in the same order: the results are the same bits,
        # and anything left in the array by the call before would show as a difference
        assert torch.equal(got, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from sandyrt_b200.csrc.build import load_library

    lib = load_library("attention_decode")
    lib.sandy_decode_attention_static_strerror.restype = ctypes.c_char_p
    H, D, page_size = 32, 128, 16
    c = _case(3, torch.bfloat16, H, D, page_size, [20] * 64)
    out = torch.zeros_like(c["q"])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # 64 tokens * 32 heads * 8 splits * 130 floats = 2,129,920 > 1,048,576
    code = _call_static(lib, c, out, H, D, page_size, 0.1, 8, status)
    assert code == -3
    assert b"more scratch than the static array holds" in lib.sandy_decode_attention_static_strerror(code)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0            # nothing was launched
    # factors so large that their product would wrap around a 64-bit integer are refused too
    for n_tokens, n_heads, splits in ((64, 32, 2 ** 31 - 1), (2 ** 31 - 1, 2 ** 31 - 1, 2 ** 31 - 1)):
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        code = lib.sandy_decode_attention_static(
            p(c["q"]), ctypes.c_int(c["q"].stride(0)), p(c["kc"]), p(c["vc"]), ctypes.c_longlong(c["kc"].stride(0)),
            p(c["table"]), ctypes.c_int(c["table"].shape[1]), p(c["tok_seq"]), p(c["tok_pos"]), p(out),
            ctypes.c_int(out.stride(0)), ctypes.c_int(n_tokens), ctypes.c_int(n_heads), ctypes.c_int(n_heads),
            ctypes.c_int(D), ctypes.c_int(page_size), ctypes.c_float(0.1), ctypes.c_int(0), ctypes.c_int(splits),
            ctypes.c_int(c["kc"].shape[0]), ctypes.c_int(1), p(status), ctypes.c_void_p(0))
        assert code == -3
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
    # the same shape with one split needs no scratch at all and runs
    assert _call_static(lib, c, out, H, D, page_size, 0.1, 1, status) == 0
    torch.cuda.synchronize()
    assert float(out.abs().sum()) > 0.0
