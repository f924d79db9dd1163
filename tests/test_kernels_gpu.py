"""Each kernel alone against a plain float32 reference of the same op, at sizes other than
the engine's: odd widths, vocabularies that are no power of two, head sizes in steps of 16,
head counts and groups that are no power of two."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _gelu_new(u):
    return 0.5 * u * (1 + torch.tanh(0.7978845608028654 * (u + 0.044715 * u ** 3)))


def _act(u, act):
    if act == "gelu_new":
        return _gelu_new(u)
    if act == "gelu":
        return 0.5 * u * (1 + torch.erf(u / math.sqrt(2.0)))
    return u


# ---- embedding ---------------------------------------------------------------------------
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,vocab,npos", [(64, 512, 128), (240, 777, 33), (1600, 1000, 50)])
def test_embed_positions(table_dtype, width, vocab, npos):
    from sandyrt_b200.csrc import ops

    wte, wpe = _rand((vocab, width), table_dtype, 1), _rand((npos, width), table_dtype, 2)
    ids = torch.randint(0, vocab, (37,), dtype=torch.int32, device=DEV)
    pos = torch.randint(0, npos, (37,), dtype=torch.int32, device=DEV)
    out = torch.empty(37, width, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_positions(ids, pos, wte, wpe, out, status=status)
    want = wte.float()[ids.long()] + wpe.float()[pos.long()]
    assert torch.equal(out, want) and int(status.item()) == 0
    # no position table
    ops.embed_positions(ids, pos, wte, None, out)
    assert torch.equal(out, wte.float()[ids.long()])
    # an id outside the table is reported, not read
    ids[5] = vocab
    ops.embed_positions(ids, pos, wte, wpe, out, status=status)
    assert int(status.item()) & 1 and float(out[5].abs().sum()) == 0.0


# ---- layernorm ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32, torch.float32),
                                    (torch.float32, torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("width,eps", [(64, 1e-5), (96, 1e-6), (240, 3e-5), (1600, 1e-5), (5000, 1e-3)])
def test_layernorm(dtypes, width, eps):
    from sandyrt_b200.csrc import ops

    tin, tw, tout = dtypes
    x = _rand((29, width), tin, 3, scale=3.0) + 1.5
    g, b = _rand((width,), tw, 4) + 1.0, _rand((width,), tw, 5)
    out = torch.empty(29, width, dtype=tout, device=DEV)
    ops.layernorm(x, g, b, eps, out)
    xd = x.double()
    mean = xd.mean(-1, keepdim=True)
    var = ((xd - mean) ** 2).mean(-1, keepdim=True)
    want = ((xd - mean) / torch.sqrt(var + eps) * g.double() + b.double())
    tol = 2e-5 if tout == torch.float32 else 2e-2
    assert (out.double() - want).abs().max().item() < tol * (1 + want.abs().max().item())
    # selected rows only
    rows = torch.tensor([28, 0, 7, 7], dtype=torch.int32, device=DEV)
    out2 = torch.empty(4, width, dtype=tout, device=DEV)
    ops.layernorm(x, g, b, eps, out2, rows=rows)
    assert torch.equal(out2, out[rows.long()])


# ---- matrix products ----------------------------------------------------------------------
def _gemm_want(a, w_kn, bias, act, residual):
    y = a.double() @ w_kn.double()
    if bias is not None:
        y = y + bias.double()
    y = _act(y, act)
    if residual is not None:
        y = y + residual.double()
    return y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 192, 64), (33, 1000, 96), (130, 320, 96), (64, 777, 240), (7, 50, 13)])
@pytest.mark.parametrize("layout", ["in_out", "out_in"])
def test_gemm_simt(dtype, M, N, K, layout):
    from sandyrt_b200.csrc import ops

    a = _rand((M, K), dtype, 1)
    w_kn = _rand((K, N), dtype, 2, scale=0.1)
    bias = _rand((N,), dtype, 3)
    res = _rand((M, N), torch.float32, 4)
    w = w_kn if layout == "in_out" else w_kn.t().contiguous()
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    for act, use_res, out_dtype in ((None, False, dtype), ("gelu_new", False, dtype), ("gelu", False, dtype),
                                    (None, True, torch.float32)):
        if dtype == torch.float32 and out_dtype != torch.float32:
            continue
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.gemm_simt(a, w, bias, out, w_out_in=(layout == "out_in"), act=act, residual=res if use_res else None)
        want = _gemm_want(a, w_kn, bias, act, res if use_res else None)
        err = (out.double() - want).abs().max().item()
        assert err < tol * (1 + want.abs().max().item()), (act, use_res, err)


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 2304, 768), (100, 777, 240), (128, 128, 64), (129, 130, 72),
                                   (300, 1000, 96), (2048, 768, 3072), (257, 320, 96), (64, 50257, 64), (517, 96, 320)])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, -64, -128, -256, 2128, 2256])
def test_gemm_tc(M, N, K, tile_n):
    """The tcgen05 kernels (positive tile widths: the persistent kernel; negative: one tile per
    CTA; 2000 + width: two CTAs on a 256-row tile) at sizes that are no multiple of their tiles,
    every epilogue."""
    from sandyrt_b200.csrc import ops

    a = _rand((M, K), torch.bfloat16, 1)
    w_nk = _rand((N, K), torch.bfloat16, 2, scale=0.1)
    bias = _rand((N,), torch.bfloat16, 3)
    res = _rand((M, N), torch.float32, 4)
    for act, use_res, out_dtype, use_bias in ((None, False, torch.bfloat16, True), ("gelu_new", False, torch.bfloat16, True),
                                              ("gelu", False, torch.bfloat16, True), (None, True, torch.float32, True),
                                              (None, False, torch.float32, False)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops.gemm_tc(a, w_nk, bias if use_bias else None, out, act=act, residual=res if use_res else None, tile_n=tile_n)
        ops.check_kernel_status(DEV)
        want = _gemm_want(a, w_nk.t(), bias if use_bias else None, act, res if use_res else None)
        tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-5
        err = (out.double() - want).abs().max().item()
        assert err < tol * (1 + want.abs().max().item()), (act, use_res, out_dtype, err)


@pytest.mark.parametrize("tile_n", [0, 128, 256, -64, -128, 2128, 2256])
@pytest.mark.parametrize("N,pitch", [(1000, 1000), (1000, 1024), (777, 777), (777, 784), (96, 4096), (40, 40)])
def test_gemm_tc_write_back_paths(tile_n, N, pitch):
    """Above one tile of rows the write-back goes through TMA stores where the output's rows start on
    16-byte boundaries (a reduce-add where the residual is the output itself) and through the registers
    where they do not; either way nothing is written outside the [M, N] window of a wider buffer, and a
    last tile that is cut by M and by N is clipped."""
    from sandyrt_b200.csrc import ops

    M, K = 300, 200
    a = _rand((M, K), torch.bfloat16, 1)
    w = _rand((N, K), torch.bfloat16, 2, scale=0.1)
    bias = _rand((N,), torch.bfloat16, 3)
    for dtype in (torch.bfloat16, torch.float32):
        wide = torch.full((M + 3, pitch), 7.0, dtype=dtype, device=DEV)
        out = wide[:M, :N]
        ops.gemm_tc(a, w, bias, out, act="gelu_new", tile_n=tile_n)
        ops.check_kernel_status(DEV)
        want = _gemm_want(a, w.t(), bias, "gelu_new", None)
        tol = 1e-2 if dtype == torch.bfloat16 else 2e-5
        assert (out.double() - want).abs().max().item() < tol * (1 + want.abs().max().item()), (dtype, "values")
        assert bool((wide[M:] == 7.0).all()) and bool((wide[:, N:] == 7.0).all()), (dtype, "wrote outside its window")
    # the residual stream: in place, twice over (every element receives exactly one addition a launch)
    wide = torch.zeros(M + 3, pitch, dtype=torch.float32, device=DEV)
    x0 = _rand((M, N), torch.float32, 4)
    wide[:M, :N] = x0
    x = wide[:M, :N]
    ops.gemm_tc(a, w, bias, x, residual=x, tile_n=tile_n)
    ops.gemm_tc(a, w, bias, x, residual=x, tile_n=tile_n)
    ops.check_kernel_status(DEV)
    want = x0.double() + 2 * (a.double() @ w.double().t() + bias.double())
    assert (x.double() - want).abs().max().item() < 1e-4 * (1 + want.abs().max().item())
    assert float(wide[M:].abs().sum()) == 0.0 and float(wide[:, N:].abs().sum()) == 0.0
    # and the same bits whichever way the tiles are cut
    y = x0.clone()
    ops.gemm_tc(a, w, bias, y, residual=y, tile_n=-128)
    ops.gemm_tc(a, w, bias, y, residual=y, tile_n=-128)
    assert torch.equal(y, x.contiguous())


def test_gemm_tc_in_place_residual_and_row_independence():
    """out may be the residual itself; a row's result does not depend on the rows beside it."""
    from sandyrt_b200.csrc import ops

    a = _rand((200, 96), torch.bfloat16, 1)
    w = _rand((96, 96), torch.bfloat16, 2, scale=0.1)
    x = _rand((200, 96), torch.float32, 3)
    want = x.double() + a.double() @ w.double().t()
    ops.gemm_tc(a, w, None, x, residual=x)
    assert (x.double() - want).abs().max().item() < 1e-4
    full = torch.empty(200, 96, dtype=torch.float32, device=DEV)
    ops.gemm_tc(a, w, None, full)
    part = torch.empty(3, 96, dtype=torch.float32, device=DEV)
    ops.gemm_tc(a[130:133].contiguous(), w, None, part)
    assert torch.equal(part, full[130:133])


def test_gemm_tc_refuses_what_it_cannot_take():
    from sandyrt_b200.csrc import ops

    a = _rand((4, 60), torch.bfloat16, 1)
    w = _rand((16, 60), torch.bfloat16, 2)
    out = torch.empty(4, 16, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.UnsupportedShape):
        ops.gemm_tc(a, w, None, out)          # K = 60 is no multiple of 8
    assert not ops.tensor_core_gemm_supported(60, 16)


# ---- attention over the paged cache ------------------------------------------------------------
def _paged_case(dtype, H, Hkv, D, page_size, seqs, seed, spike=None, runs=(), swap=None):
    """seqs: list of (tokens already cached, new tokens).  Builds q for the new tokens, dense
    K/V per request, and a cache whose pages are handed out in a shuffled order; the cached
    prefix is written directly, the new tokens' K/V through kv_append.  `spike`: (request,
    key position): that key and every query of the request are scaled so that this one score
    stands out among hundreds.  `runs`: requests whose pages follow one another in the cache (the
    way a pool hands them out to a prompt), instead of lying anywhere; `swap`: (request, i, j): its
    blocks i and j change pages, which breaks a run inside a key tile."""
    from sandyrt_b200.csrc import ops

    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blocks = [-(-(b + n) // page_size) for b, n in seqs]
    num_pages = sum(n_blocks) + 3
    n_run = sum(n_blocks[s] for s in runs)
    run_first = 1                                          # runs lie at pages 1 .. n_run, the others anywhere behind
    perm = (torch.randperm(num_pages - n_run - 1, generator=g) + n_run + 1).tolist() + [0]
    max_blocks = max(n_blocks) + 2
    table = torch.full((len(seqs), max_blocks), -1, dtype=torch.int32)
    arena = torch.full((num_pages, 2, Hkv, page_size, D), float("nan"), dtype=dtype)
    dense_k, dense_v, qs, tok_seq, tok_pos, k_new, v_new = [], [], [], [], [], [], []
    for s, (before, n) in enumerate(seqs):
        L = before + n
        k = torch.randn(L, Hkv, D, generator=g)
        v = torch.randn(L, Hkv, D, generator=g)
        q = torch.randn(n, H, D, generator=g)
        if spike is not None and spike[0] == s:
            k[spike[1]] *= 6.0
            q = q.abs() * torch.sign(k[spike[1]]).repeat_interleave(H // Hkv, dim=0) * 1.5
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        dense_k.append(k); dense_v.append(v); qs.append(q)
        for b in range(n_blocks[s]):
            if s in runs:
                table[s, b] = run_first
                run_first += 1
            else:
                table[s, b] = perm.pop()
        if swap is not None and swap[0] == s:
            i, j = swap[1], swap[2]
            table[s, i], table[s, j] = table[s, j].clone(), table[s, i].clone()
        for p in range(before):
            page = table[s, p // page_size]
            arena[page, 0, :, p % page_size] = k[p]
            arena[page, 1, :, p % page_size] = v[p]
        tok_seq += [s] * n
        tok_pos += list(range(before, L))
        k_new.append(k[before:]); v_new.append(v[before:])
    arena = arena.to(DEV)
    kc, vc = arena[:, 0], arena[:, 1]
    table = table.to(DEV)
    tok_seq = torch.tensor(tok_seq, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(tok_pos, dtype=torch.int32, device=DEV)
    kv_src = torch.cat([torch.cat(k_new).reshape(-1, Hkv * D), torch.cat(v_new).reshape(-1, Hkv * D)], dim=1).to(DEV)
    ops.kv_append(kv_src[:, :Hkv * D], kv_src[:, Hkv * D:], kc, vc, table, tok_seq, tok_pos)
    q_all = torch.cat(qs).reshape(-1, H * D).to(DEV)
    return dict(q=q_all, kc=kc, vc=vc, table=table, tok_seq=tok_seq, tok_pos=tok_pos,
                dense_k=dense_k, dense_v=dense_v, qs=qs, seqs=seqs)


def _attention_want(case, H, Hkv, D, scale, window):
    outs = []
    for s, (before, n) in enumerate(case["seqs"]):
        k, v, q = case["dense_k"][s].double(), case["dense_v"][s].double(), case["qs"][s].double()
        for i in range(n):
            pos = before + i
            lo = max(0, pos + 1 - window) if window else 0
            row = []
            for h in range(H):
                kh = h // (H // Hkv)
                sc = (k[lo:pos + 1, kh] @ q[i, h]) * scale
                p = torch.softmax(sc, dim=0)
                row.append(p @ v[lo:pos + 1, kh])
            outs.append(torch.cat(row))
    return torch.stack(outs)


ATT_TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,D,page_size,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (5, 5, 48, 8, 0),
                                                     (6, 2, 64, 16, 0), (5, 1, 80, 4, 0), (4, 2, 128, 32, 0),
                                                     (3, 3, 32, 16, 20), (6, 3, 64, 8, 37), (2, 1, 256, 16, 0)])
def test_paged_attention_general(dtype, H, Hkv, D, page_size, window):
    from sandyrt_b200.csrc import ops

    seqs = [(0, 33), (40, 1), (17, 24), (0, 1), (63, 2), (100, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=D + H)
    out = torch.full_like(case["q"], float("nan"))
    scale = 0.7 / math.sqrt(D)
    ops.paged_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out,
                        n_heads=H, scale=scale, window=window)
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert (out.double().cpu() - want).abs().max().item() < ATT_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,D,page_size,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (12, 12, 64, 16, 0),
                                                     (6, 2, 64, 8, 0), (4, 1, 128, 32, 0), (5, 5, 64, 16, 100)])
@pytest.mark.parametrize("splits", [1, 2, 5])
def test_decode_attention_split_kv(dtype, H, Hkv, D, page_size, window, splits):
    """Single tokens over contexts of 1 to 700 keys, the keys split over several blocks."""
    from sandyrt_b200.csrc import ops

    seqs = [(699, 1), (0, 1), (63, 1), (64, 1), (300, 1), (15, 1), (128, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=D + splits)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    T = case["q"].shape[0]
    scratch = torch.full((T * H * splits * (D + 2),), float("nan"), dtype=torch.float32, device=DEV)
    ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out,
                         n_heads=H, scale=scale, window=window, num_splits=splits, scratch=scratch)
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert (out.double().cpu() - want).abs().max().item() < ATT_TOL[dtype]
    # the same splits as one cluster, merged through distributed shared memory: same numbers
    if splits > 1:
        out2 = torch.full_like(case["q"], float("nan"))
        ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out2,
                             n_heads=H, scale=scale, window=window, num_splits=splits, cluster=True)
        ops.check_kernel_status(DEV)
        assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,D,page_size,window", [(4, 4, 16, 16, 0), (3, 3, 32, 64, 0), (12, 12, 64, 16, 0),
                                                     (6, 2, 64, 8, 0), (4, 1, 128, 32, 0), (5, 5, 64, 16, 100),
                                                     (2, 2, 32, 128, 0), (3, 1, 32, 4, 9)])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_decode_attention_bulk(dtype, H, Hkv, D, page_size, window, splits):
    """The variant that streams pages through a shared-memory ring: contexts of 1 to 700 keys
    (more pages than the ring has stages, so stages are used again), splits at page edges."""
    from sandyrt_b200.csrc import ops

    seqs = [(699, 1), (0, 1), (63, 1), (64, 1), (300, 1), (15, 1), (128, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=D + splits)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out,
                         n_heads=H, scale=scale, window=window, num_splits=splits, bulk=True)
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert (out.double().cpu() - want).abs().max().item() < ATT_TOL[dtype]


@pytest.mark.parametrize("H,Hkv,page_size,window", [(12, 12, 16, 0), (6, 2, 8, 0), (5, 5, 16, 100), (3, 1, 4, 9),
                                                   (2, 2, 64, 0), (4, 4, 16, 333)])
@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
def test_decode_attention_mma(H, Hkv, page_size, window, splits):
    """The variant whose products are mma.sync instructions (bfloat16, heads of 64): contexts of 1 to
    700 keys (tiles of 64 keys: more tiles than stages, last tiles partly filled, ranges that begin and
    end inside a tile), grouped heads, windows, every split count; and slots of the cache that hold no
    key of the request are poisoned, so a weight of zero that met one would show."""
    from sandyrt_b200.csrc import ops

    D, dtype = 64, torch.bfloat16
    seqs = [(699, 1), (0, 1), (63, 1), (64, 1), (300, 1), (15, 1), (128, 1), (65, 1), (511, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=7 + splits)
    # poison every slot behind a request's last position and every page no request holds
    kc, vc, table = case["kc"], case["vc"], case["table"].cpu()
    used = torch.zeros(kc.shape[0], page_size, dtype=torch.bool)
    for s_i, (before, n) in enumerate(seqs):
        for pos in range(before + n):
            used[int(table[s_i, pos // page_size]), pos % page_size] = True
    mask = (~used).to(DEV)[:, None, :, None].expand(-1, Hkv, -1, D)
    kc[mask] = float("nan")
    vc[mask] = float("inf")
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    run = lambda: ops.decode_attention(case["q"], kc, vc, case["table"], case["tok_seq"], case["tok_pos"], out,
                                       n_heads=H, scale=scale, window=window, num_splits=splits, mma=True)
    if case["table"].shape[1] * page_size > (160 - 2) * page_size * splits:
        # a block keeps the page numbers of its range in shared memory: more pages than it holds are refused
        with pytest.raises(ops.UnsupportedShape):
            run()
        return
    run()
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert bool(torch.isfinite(out.float()).all())
    assert (out.double().cpu() - want).abs().max().item() < ATT_TOL[dtype]


@pytest.mark.parametrize("kernel", ["general", "decode", "bulk", "mma"])
def test_one_far_key_among_hundreds(kernel):
    """Scale one query/key pair so that a single score dominates: a kernel that dropped or
    misplaced that key (a page's edge, a split's edge) returns a visibly different output."""
    from sandyrt_b200.csrc import ops

    H = Hkv = 2
    D = 64
    # pages of 16 and pages of 4 (a block table of 161 entries)
    for far, ps in ((0, 16), (15, 16), (16, 16), (255, 16), (256, 16), (399, 16), (511, 16), (640, 16),
                    (0, 4), (255, 4), (257, 4), (640, 4)):
        seqs = [(641, 1), (5, 1)]
        case = _paged_case(torch.bfloat16 if kernel == "mma" else torch.float32, H, Hkv, D, ps, seqs, seed=far, spike=(0, far))
        out = torch.full_like(case["q"], float("nan"))
        if kernel == "mma":
            ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"],
                                 out, n_heads=H, scale=0.125, num_splits=7, mma=True)
            got = out[0].view(H, D).float().cpu()
            v_far = case["dense_v"][0][far].float()
            assert (got - v_far).abs().max().item() < 3e-2, f"far key {far}: output is not that key's value"
            continue
        if kernel == "general":
            ops.paged_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"],
                                out, n_heads=H, scale=0.125)
        elif kernel == "bulk":
            ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"],
                                 out, n_heads=H, scale=0.125, num_splits=7, bulk=True)
        else:
            scratch = torch.empty(2 * H * 7 * (D + 2), dtype=torch.float32, device=DEV)
            ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"],
                                 out, n_heads=H, scale=0.125, num_splits=7, scratch=scratch)
        got = out[0].view(H, D).cpu()
        v_far = case["dense_v"][0][far]
        assert (got - v_far).abs().max().item() < 1e-3, f"far key {far}: output is not that key's value"
        want = _attention_want(case, H, Hkv, D, 0.125, 0)
        assert (out.double().cpu() - want).abs().max().item() < 2e-5


@pytest.mark.parametrize("H,Hkv,D,page_size,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (5, 5, 48, 8, 0),
                                                     (12, 12, 64, 16, 0), (6, 2, 64, 16, 0), (5, 1, 80, 4, 0),
                                                     (4, 2, 128, 32, 0), (3, 3, 32, 16, 20), (6, 3, 64, 8, 70),
                                                     (2, 2, 96, 16, 0), (2, 1, 112, 16, 0)])
@pytest.mark.parametrize("tc", [None, False])
def test_prefill_attention_tensor_cores(H, Hkv, D, page_size, window, tc):
    """tc None: heads of 64 on the tcgen05 kernel, the others on the mma.sync kernel; False: all
    on the mma.sync kernel.  Portions that start at 0 and in the middle of a prompt, of 1 to 200 tokens, beside
    single tokens; tile edges (63/64/65), page edges, windows."""
    from sandyrt_b200.csrc import ops

    seqs = [(0, 200), (40, 1), (17, 64), (0, 1), (63, 65), (100, 2), (0, 63), (129, 130)]
    case = _paged_case(torch.bfloat16, H, Hkv, D, page_size, seqs, seed=D + H)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    lens = [n for _, n in seqs]
    q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    kv_before = torch.tensor([b for b, _ in seqs], dtype=torch.int32, device=DEV)
    ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                          max_q_len=max(lens), scale=scale, window=window, tc=tc)
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert not torch.isnan(out).any()
    assert (out.double().cpu() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("H,Hkv,D,page_size,window", [(3, 3, 64, 16, 0), (4, 2, 32, 16, 0), (2, 2, 128, 32, 0),
                                                     (3, 1, 64, 8, 150)])
@pytest.mark.parametrize("tc", [None, False])
def test_prefill_attention_long_portions(H, Hkv, D, page_size, window, tc):
    """Portions of 256 tokens and more (many key tiles per query tile): a portion from position 0,
    one behind a long prefix, an odd number of tiles, short ones beside them, a window."""
    from sandyrt_b200.csrc import ops

    seqs = [(0, 700), (300, 257), (0, 64), (50, 1), (1000, 320)]
    case = _paged_case(torch.bfloat16, H, Hkv, D, page_size, seqs, seed=D + H)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    lens = [n for _, n in seqs]
    q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    kv_before = torch.tensor([b for b, _ in seqs], dtype=torch.int32, device=DEV)
    ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                          max_q_len=max(lens), scale=scale, window=window, tc=tc)
    ops.check_kernel_status(DEV)
    want = _attention_want(case, H, Hkv, D, scale, window)
    assert not torch.isnan(out).any()
    assert (out.double().cpu() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("H,Hkv,page_size,window", [(3, 3, 16, 0), (4, 2, 8, 0), (2, 1, 32, 200), (2, 2, 64, 0),
                                                   (2, 2, 128, 0)])
def test_prefill_attention_page_runs(H, Hkv, page_size, window):
    """Requests whose pages follow one another in the cache beside requests whose pages lie anywhere:
    the tcgen05 kernel fetches whole key tiles of the former with TMA and the rest (and every
    request's last, partly filled tile) with copies by its threads.  Portions at position 0 and
    behind a prefix, aligned to the tiles and not, a far key in a tile that TMA fetched."""
    from sandyrt_b200.csrc import ops

    D = 64
    seqs = [(0, 512), (256, 300), (0, 700), (130, 257), (0, 128), (384, 1)]
    for far in (5, 300):
        case = _paged_case(torch.bfloat16, H, Hkv, D, page_size, seqs, seed=H + page_size, runs=(0, 1, 4, 5),
                           spike=(0, far))
        out = torch.full_like(case["q"], float("nan"))
        scale = 1.0 / math.sqrt(D)
        lens = [n for _, n in seqs]
        q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
        kv_before = torch.tensor([b for b, _ in seqs], dtype=torch.int32, device=DEV)
        ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                              max_q_len=max(lens), scale=scale, window=window, tc=True)
        ops.check_kernel_status(DEV)
        want = _attention_want(case, H, Hkv, D, scale, window)
        assert not torch.isnan(out).any()
        assert (out.double().cpu() - want).abs().max().item() < 2e-2
        if window == 0:
            v_far = case["dense_v"][0][far].float().repeat_interleave(H // Hkv, dim=0)
            got = out[max(far, 0):512].view(-1, H, D).float().cpu()
            assert (got - v_far).abs().max().item() < 3e-2, f"far key {far}"


def test_prefill_attention_broken_run_and_long_tables():
    """A run of pages with two pages exchanged (tiles with the break come by the threads' copies,
    the others by TMA); a block table longer than the kernel keeps in shared memory; more key tiles
    than it keeps run marks for."""
    from sandyrt_b200.csrc import ops

    H, Hkv, D = 2, 1, 64
    for page_size, seqs, runs, swap in ((16, [(0, 600), (100, 3)], (0,), (0, 3, 20)),
                                        (8, [(9000, 130), (0, 64)], (0, 1), None),
                                        (16, [(16500, 130)], (0,), None)):
        case = _paged_case(torch.bfloat16, H, Hkv, D, page_size, seqs, seed=page_size, runs=runs, swap=swap)
        out = torch.full_like(case["q"], float("nan"))
        scale = 1.0 / math.sqrt(D)
        lens = [n for _, n in seqs]
        q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
        kv_before = torch.tensor([b for b, _ in seqs], dtype=torch.int32, device=DEV)
        ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                              max_q_len=max(lens), scale=scale, tc=True)
        ops.check_kernel_status(DEV)
        want = _attention_want(case, H, Hkv, D, scale, 0)
        assert not torch.isnan(out).any()
        assert (out.double().cpu() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("tc", [None, False])
def test_prefill_attention_far_key(tc):
    from sandyrt_b200.csrc import ops

    H = Hkv = 2
    D = 64
    for far in (0, 63, 64, 127, 300, 511, 512):
        seqs = [(520, 90), (5, 3)]
        case = _paged_case(torch.bfloat16, H, Hkv, D, 16, seqs, seed=far, spike=(0, far))
        out = torch.full_like(case["q"], float("nan"))
        q_start = torch.tensor([0, 90, 93], dtype=torch.int32, device=DEV)
        kv_before = torch.tensor([520, 5], dtype=torch.int32, device=DEV)
        ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                              max_q_len=90, scale=0.125, tc=tc)
        v_far = case["dense_v"][0][far].float()
        got = out[:90].view(90, H, D).float().cpu()
        assert (got - v_far).abs().max().item() < 3e-2, f"far key {far}"
        # the same with a long portion (five query tiles, up to ten key tiles each)
        seqs = [(310, 300), (5, 3)]
        case = _paged_case(torch.bfloat16, H, Hkv, D, 16, seqs, seed=far, spike=(0, far))
        out = torch.full_like(case["q"], float("nan"))
        q_start = torch.tensor([0, 300, 303], dtype=torch.int32, device=DEV)
        kv_before = torch.tensor([310, 5], dtype=torch.int32, device=DEV)
        ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                              max_q_len=300, scale=0.125, tc=tc)
        ops.check_kernel_status(DEV)
        if far <= 310:          # visible to every query of the portion
            v_far = case["dense_v"][0][far].float()
            got = out[:300].view(300, H, D).float().cpu()
            assert (got - v_far).abs().max().item() < 3e-2, f"far key {far}, long portion"


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(64, 64), (2304, 768), (777, 240), (50257, 64), (16401, 776), (96, 320), (1000, 96),
                                 (13, 8), (4800, 1600), (1304, 2056)])     # the last two: more blocks than SMs and a long K
def test_gemm_skinny(M, N, K):
    """The decode-step product at 1..64 rows, odd N, K that is no multiple of its 32-wide chunks;
    with very many columns, up to 16 rows and nothing fused the kernel whose warps walk the column
    groups takes it."""
    from sandyrt_b200.csrc import ops

    a = _rand((M, K), torch.bfloat16, 1)
    w_nk = _rand((N, K), torch.bfloat16, 2, scale=0.1)
    bias = _rand((N,), torch.bfloat16, 3)
    res = _rand((M, N), torch.float32, 4)
    for act, use_res, out_dtype, use_bias in ((None, False, torch.bfloat16, True), ("gelu_new", False, torch.bfloat16, True),
                                              ("gelu", False, torch.bfloat16, True), (None, True, torch.float32, True),
                                              (None, False, torch.float32, False)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops.gemm_skinny(a, w_nk, bias if use_bias else None, out, act=act, residual=res if use_res else None)
        want = _gemm_want(a, w_nk.t(), bias if use_bias else None, act, res if use_res else None)
        tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-5
        err = (out.double() - want).abs().max().item()
        assert err < tol * (1 + want.abs().max().item()), (act, use_res, out_dtype, err)
    # in place on the residual
    x = res.clone()
    ops.gemm_skinny(a, w_nk, None, x, residual=x)
    assert (x.double() - (res.double() + a.double() @ w_nk.double().t())).abs().max().item() < 1e-4


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("K,N,eps", [(64, 192, 1e-5), (768, 2304, 1e-5), (96, 320, 1e-6), (240, 777, 3e-5), (1600, 136, 1e-5), (2048, 64, 1e-5)])
def test_gemm_skinny_with_the_norm_inside(M, K, N, eps):
    """LayerNorm run inside the product equals the stand-alone norm kernel followed by the product."""
    from sandyrt_b200.csrc import ops

    x = _rand((M, K), torch.float32, 1, scale=2.0) + 0.3
    norm = lazy = ops.FusedNorm(x, _rand((K,), torch.bfloat16, 4) + 1.0, _rand((K,), torch.bfloat16, 5), eps)
    w = _rand((N, K), torch.bfloat16, 2, scale=0.1)
    bias = _rand((N,), torch.bfloat16, 3)
    assert ops.skinny_norm_fusable(lazy, K)
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(None, w, bias, got, act="gelu_new", norm=lazy)
    h = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    ops.layernorm(x, norm.gamma, norm.beta, eps, h)
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(h, w, bias, want, act="gelu_new")
    # the two norms add in another order: an element of h may round the other way now and then
    assert (got.float() - want.float()).abs().max().item() < 2e-2 * (1 + want.float().abs().max().item())
    xd = x.double()
    hd = ((xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + eps)
          * norm.gamma.double() + norm.beta.double())
    ref = _gemm_want(hd, w.t(), bias, "gelu_new", None)
    assert (got.double() - ref).abs().max().item() < 2e-2 * (1 + ref.abs().max().item())


@pytest.mark.parametrize("H,Hkv,D,seqs", [
    (6, 2, 32, [(13, 1), (0, 1), (7, 1), (40, 1), (8, 3)]),
    # 40 rows and 1,792 columns: the form with sixteen columns a block, three row tiles
    (12, 8, 64, [(13, 1), (0, 30), (7, 1), (40, 1), (8, 7)]),
])
def test_gemm_skinny_writes_keys_and_values_into_the_pages(H, Hkv, D, seqs):
    """The fused q/k/v product puts its key and value columns where kv_append would."""
    from sandyrt_b200.csrc import ops
    from sandyrt_b200.csrc.ops import KVTarget

    ps = 8
    q_cols, kv_cols = H * D, Hkv * D
    K = 96
    T = sum(n for _, n in seqs)
    num_pages = 32
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(seqs), 8), -1, dtype=torch.int32)
    tok_seq, tok_pos = [], []
    for s, (before, n) in enumerate(seqs):
        for b in range(-(-(before + n) // ps)):
            table[s, b] = perm.pop()
        tok_seq += [s] * n
        tok_pos += list(range(before, before + n))
    table = table.to(DEV)
    tok_seq = torch.tensor(tok_seq, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(tok_pos, dtype=torch.int32, device=DEV)
    a = _rand((T, K), torch.bfloat16, 1)
    w = _rand((q_cols + 2 * kv_cols, K), torch.bfloat16, 2, scale=0.2)
    bias = _rand((q_cols + 2 * kv_cols,), torch.bfloat16, 3)
    arena_a = torch.zeros(num_pages, 2, Hkv, ps, D, dtype=torch.bfloat16, device=DEV)
    arena_b = torch.zeros_like(arena_a)
    out_a = torch.empty(T, q_cols + 2 * kv_cols, dtype=torch.bfloat16, device=DEV)
    out_b = torch.empty_like(out_a)
    target = KVTarget(arena_a[:, 0], arena_a[:, 1], table, tok_seq, tok_pos, q_cols, kv_cols, D)
    ops.gemm_skinny(a, w, bias, out_a, kv=target)
    ops.gemm_skinny(a, w, bias, out_b)
    ops.kv_append(out_b[:, q_cols:q_cols + kv_cols], out_b[:, q_cols + kv_cols:], arena_b[:, 0], arena_b[:, 1],
                  table, tok_seq, tok_pos)
    ops.check_kernel_status(DEV)
    assert torch.equal(out_a, out_b)
    assert torch.equal(arena_a, arena_b) and float(arena_a.abs().sum()) > 0


@pytest.mark.parametrize("M", [1, 17, 24, 32, 33, 47, 64, 65, 128, 200, 256])
@pytest.mark.parametrize("N,K", [(64, 64), (2304, 768), (768, 3072), (777, 240), (50257, 64), (16401, 776), (96, 320),
                                 (1000, 96), (13, 8), (136, 1600), (520, 4104)])
def test_gemm_small(M, N, K):
    """The product of 17..64 rows on tcgen05 with the weight as the wide operand: one block a tile
    and clusters of 2 to 8 blocks that split K (which of them depends on the shape), odd N, a K
    that is no multiple of the 64-wide k-step, rows that do not fill the instruction's 64."""
    from sandyrt_b200.csrc import ops

    a = _rand((M, K), torch.bfloat16, 1)
    w_nk = _rand((N, K), torch.bfloat16, 2, scale=0.1)
    bias = _rand((N,), torch.bfloat16, 3)
    res = _rand((M, N), torch.float32, 4)
    for act, use_res, out_dtype, use_bias in ((None, False, torch.bfloat16, True), ("gelu_new", False, torch.bfloat16, True),
                                              (None, True, torch.float32, True), (None, False, torch.float32, False)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops.gemm_small(a, w_nk, bias if use_bias else None, out, act=act, residual=res if use_res else None)
        ops.check_kernel_status(DEV)
        want = _gemm_want(a, w_nk.t(), bias if use_bias else None, act, res if use_res else None)
        tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-5
        err = (out.double() - want).abs().max().item()
        assert err < tol * (1 + want.abs().max().item()), (act, use_res, out_dtype, err, ops.gemm_small_splits(N, K))
    # in place on the residual, and the same bits every time (the blocks' sums are added in a fixed order)
    x = res.clone()
    ops.gemm_small(a, w_nk, None, x, residual=x)
    assert (x.double() - (res.double() + a.double() @ w_nk.double().t())).abs().max().item() < 1e-4
    first = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_small(a, w_nk, bias, first)
    for _ in range(3):
        again = torch.empty_like(first)
        ops.gemm_small(a, w_nk, bias, again)
        assert torch.equal(first, again)


def test_gemm_small_splits_are_a_rule_of_the_shape():
    from sandyrt_b200.csrc import ops

    seen = {ops.gemm_small_splits(N, K) for N, K in ((2304, 768), (768, 3072), (50257, 768), (64, 64), (768, 768))}
    assert all(1 <= s <= 8 for s in seen) and 1 in seen and max(seen) > 1
    assert ops.gemm_small_splits(50257, 768) == 1            # more tiles than SMs: nothing to split
    assert ops.gemm_small_splits(64, 64) == 1                # one k-step


@pytest.mark.parametrize("H,Hkv,D,ps,K", [(6, 2, 32, 8, 96), (3, 3, 16, 16, 512), (5, 1, 48, 4, 1280)])
def test_gemm_small_writes_keys_and_values_into_the_pages(H, Hkv, D, ps, K):
    """The fused q/k/v product of a decode step of 17..64 requests puts its key and value columns where
    kv_append would (split and unsplit K)."""
    from sandyrt_b200.csrc import ops
    from sandyrt_b200.csrc.ops import KVTarget

    q_cols, kv_cols = H * D, Hkv * D
    g = torch.Generator().manual_seed(0)
    befores = torch.randint(0, 60, (37,), generator=g).tolist()
    seqs = [(b, 1) for b in befores] + [(8, 3), (ps - 1, 2)]
    T = sum(n for _, n in seqs)
    max_blocks = -(-64 // ps)
    num_pages = len(seqs) * max_blocks + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(seqs), max_blocks), -1, dtype=torch.int32)
    tok_seq, tok_pos = [], []
    for s, (before, n) in enumerate(seqs):
        for b in range(-(-(before + n) // ps)):
            table[s, b] = perm.pop()
        tok_seq += [s] * n
        tok_pos += list(range(before, before + n))
    table = table.to(DEV)
    tok_seq = torch.tensor(tok_seq, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(tok_pos, dtype=torch.int32, device=DEV)
    a = _rand((T, K), torch.bfloat16, 1)
    w = _rand((q_cols + 2 * kv_cols, K), torch.bfloat16, 2, scale=0.2)
    bias = _rand((q_cols + 2 * kv_cols,), torch.bfloat16, 3)
    arena_a = torch.zeros(num_pages, 2, Hkv, ps, D, dtype=torch.bfloat16, device=DEV)
    arena_b = torch.zeros_like(arena_a)
    out_a = torch.empty(T, q_cols + 2 * kv_cols, dtype=torch.bfloat16, device=DEV)
    out_b = torch.empty_like(out_a)
    target = KVTarget(arena_a[:, 0], arena_a[:, 1], table, tok_seq, tok_pos, q_cols, kv_cols, D)
    ops.gemm_small(a, w, bias, out_a, kv=target)
    ops.gemm_small(a, w, bias, out_b)
    ops.kv_append(out_b[:, q_cols:q_cols + kv_cols], out_b[:, q_cols + kv_cols:], arena_b[:, 0], arena_b[:, 1],
                  table, tok_seq, tok_pos)
    ops.check_kernel_status(DEV)
    assert torch.equal(out_a, out_b)
    assert torch.equal(arena_a, arena_b) and float(arena_a.abs().sum()) > 0


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, -64, -128, -256, 2128, 2256])
@pytest.mark.parametrize("H,Hkv,D,ps", [(6, 2, 32, 8), (3, 3, 16, 16), (5, 1, 48, 4)])
def test_gemm_tc_writes_keys_and_values_into_the_pages(tile_n, H, Hkv, D, ps):
    """The fused q/k/v product of a prompt step on tcgen05 with the cache write in its write-back:
    same product, same pages as the product followed by kv_append.  Portions of several requests
    (one behind a prefix, tokens that cross page edges), column ranges that are no multiple of
    the kernel's 32-column chunks."""
    from sandyrt_b200.csrc import ops
    from sandyrt_b200.csrc.ops import KVTarget

    q_cols, kv_cols = H * D, Hkv * D
    K = 96
    seqs = [(13, 150), (0, 77), (7, 1), (40, 200)]
    T = sum(n for _, n in seqs)
    num_pages = 160
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(-(-(b + n) // ps) for b, n in seqs)
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    tok_seq, tok_pos = [], []
    for s, (before, n) in enumerate(seqs):
        for b in range(-(-(before + n) // ps)):
            table[s, b] = perm.pop()
        tok_seq += [s] * n
        tok_pos += list(range(before, before + n))
    table = table.to(DEV)
    tok_seq = torch.tensor(tok_seq, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(tok_pos, dtype=torch.int32, device=DEV)
    a = _rand((T, K), torch.bfloat16, 1)
    w = _rand((q_cols + 2 * kv_cols, K), torch.bfloat16, 2, scale=0.2)
    bias = _rand((q_cols + 2 * kv_cols,), torch.bfloat16, 3)
    arena_a = torch.zeros(num_pages, 2, Hkv, ps, D, dtype=torch.bfloat16, device=DEV)
    arena_b = torch.zeros_like(arena_a)
    out_a = torch.empty(T, q_cols + 2 * kv_cols, dtype=torch.bfloat16, device=DEV)
    out_b = torch.empty_like(out_a)
    target = KVTarget(arena_a[:, 0], arena_a[:, 1], table, tok_seq, tok_pos, q_cols, kv_cols, D)
    ops.gemm_tc(a, w, bias, out_a, kv=target, tile_n=tile_n)
    ops.gemm_tc(a, w, bias, out_b, tile_n=tile_n)
    ops.kv_append(out_b[:, q_cols:q_cols + kv_cols], out_b[:, q_cols + kv_cols:], arena_b[:, 0], arena_b[:, 1],
                  table, tok_seq, tok_pos)
    ops.check_kernel_status(DEV)
    assert torch.equal(out_a, out_b)
    assert torch.equal(arena_a, arena_b) and float(arena_a.abs().sum()) > 0
