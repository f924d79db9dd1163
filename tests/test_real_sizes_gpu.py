"""The engine against the plain implementation at GPT-2's real layer sizes.

The tiny configurations never reach the kernels and schedules that the real sizes pick: the
tcgen05 prompt attention (heads of 64, several key tiles, runs of pages), the tuned tcgen05
GEMM variants (256 rows and more), the bulk decode attention (256 (token, head) pairs and
more), the walking vocabulary projection at 50,257 columns, the 17..64-row product choice,
decode at 25 heads.  Two models with random weights stand for them here:

  small-2L  2 layers of GPT-2 small (width 768, 12 heads of 64, inner 3072, vocabulary 50257)
  xl-1L     1 layer of GPT-2 XL (width 1600, 25 heads of 64, inner 6400), vocabulary 2048

Random weights of N(0, 0.02) give almost flat attention, under which a wrong key, page or
split would hardly show.  So the query and key columns of every c_attn matrix are scaled by 3
after the folder is written: scores then spread over several units and every logit depends on
which keys were read.  The plain implementation reads the same folder.

Tolerances are those of tests/test_replay_gpu.py, stated relative to the size of the logits: the
bfloat16 bound there, 6e-3 absolute, is 3 % of the tiny models' logits (about 0.2 in size); the
logits of these wider models are about 0.6 to 0.8 in size, and 3 % of that is what is allowed
here.  (For scale: the plain implementation in bfloat16 and in float32 differ by up to 6e-2 on
xl-1L's logits, from rounding alone.)  The float32 bound is used as it is.
"""
import json
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from test_replay_gpu import STORE, TOL
from test_replay_gpu import _close as _close_tiny

pytestmark = pytest.mark.gpu

REAL = {
    "small-2L": dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=768, n_head=12,
                     n_inner=3072, vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                     activation_function="gelu_new", tie_word_embeddings=True),
    "xl-1L": dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=1, n_embd=1600, n_head=25,
                  n_inner=6400, vocab_size=2048, n_positions=1024, layer_norm_epsilon=1e-5,
                  activation_function="gelu_new", tie_word_embeddings=True),
}
QK_SCALE = 3.0
TINY_LOGIT_SIZE = 0.2      # root mean square of the tiny models' logits, which TOL's absolute part was set for


def _close(got, want, dtype, what):
    """test_replay_gpu's comparison, with the absolute part of the bfloat16 bound kept at the same
    fraction of the logits' size."""
    if dtype == "float32":
        return _close_tiny(got, want, dtype, what)
    got = np.asarray(got, dtype=np.float32)
    size = float(np.sqrt(np.mean(np.square(want, dtype=np.float64))))
    atol = TOL[dtype]["atol"] * max(1.0, size / TINY_LOGIT_SIZE)
    err = np.abs(got - want)
    bound = atol + TOL[dtype]["rtol"] * np.abs(want)
    if not (err <= bound).all():
        bad = np.argwhere(err > bound)[0]
        raise AssertionError(f"{what}: first wrong logit at row {bad[0]} col {bad[1]}: got {got[tuple(bad)]}, "
                             f"want {want[tuple(bad)]}, max err {err.max():.3e}, allowed {atol:.3e} + 2 %")


def _sharpen(model_dir, cfg):
    """Scale the query and key columns of every c_attn (weight and bias) by QK_SCALE."""
    from sandyrt_b200.weights.safetensors import SafetensorsFile, write_safetensors

    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    E = cfg["n_embd"]
    for i in range(cfg["n_layer"]):
        tensors[f"h.{i}.attn.c_attn.weight"][:, :2 * E] *= QK_SCALE
        tensors[f"h.{i}.attn.c_attn.bias"][:2 * E] *= QK_SCALE
    del f
    write_safetensors(path, tensors)


@pytest.fixture(scope="module")
def real_dirs(tmp_path_factory):
    from conftest import make_model_dir

    base = tmp_path_factory.mktemp("real")
    out = {}
    for i, (name, raw) in enumerate(REAL.items()):
        d = make_model_dir(raw, str(base / name), seed=41 + i)
        _sharpen(d, raw)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def real_plain(real_dirs):
    cache = {}

    def get(name, store):
        if (name, store) not in cache:
            cache[(name, store)] = plain.PlainGPT2(real_dirs[name], store=store)
        return cache[(name, store)]

    return get


def _engine(model_dir, dtype, max_tokens, max_requests=32, page_size=16):
    from sandyrt_b200.engine.step import Engine
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dir, device="cuda:0", dtype=getattr(torch, dtype))
    eng = Engine(model, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests)
    eng.cache.device_caches.poison()
    return eng


def _ids(name, n, seed):
    return np.random.default_rng(seed).integers(0, REAL[name]["vocab_size"], size=n).tolist()


# rows of a 600-token prompt worth looking at: the first, the edges of the 128-wide query and key
# tiles, page edges, the last
ROWS_600 = [0, 1, 15, 16, 63, 64, 127, 128, 129, 255, 256, 383, 384, 511, 512, 555, 598, 599]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small-2L", "xl-1L"])
def test_long_prompt_whole_and_in_portions_beside_decoding(real_dirs, real_plain, name, dtype):
    """(i) a 600-token prompt in one step; (ii) the same prompt as 300 + 257 + 43 beside a second
    request that brings a short prompt and then single tokens, 24 in all."""
    from sandyrt_b200.engine.step import StepEntry

    eng = _engine(real_dirs[name], dtype, max_tokens=1024)
    oracle = real_plain(name, STORE[dtype])
    ids = _ids(name, 600, seed=1)
    want = oracle.logits(ids, rows=ROWS_600)
    got = eng.step([StepEntry("whole", ids, ROWS_600)]).cpu().numpy()
    eng.check_status()
    _close(got, want, dtype, f"{name} whole prompt of 600")
    eng.release("whole")

    other = _ids(name, 17 + 24, seed=2)
    want_other = oracle.logits(other)
    got_rows, got_other = {}, []
    cuts = [300, 257, 43]
    pos, fed_other = 0, 0
    for step, n in enumerate(cuts):
        rows_here = [r - pos for r in ROWS_600 if pos <= r < pos + n]
        m = 17 if step == 0 else 1
        out = eng.step([StepEntry("cut", ids[pos:pos + n], rows_here),
                        StepEntry("other", other[fed_other:fed_other + m], list(range(m)))]).cpu().numpy()
        for j, r in enumerate(rows_here):
            got_rows[r + pos] = out[j].copy()
        got_other.append(out[len(rows_here):].copy())
        pos += n
        fed_other += m
    while fed_other < len(other):
        got_other.append(eng.step([StepEntry("other", other[fed_other:fed_other + 1], [0])]).cpu().numpy().copy())
        fed_other += 1
    eng.check_status()
    _close(np.stack([got_rows[r] for r in ROWS_600]), want, dtype, f"{name} prompt as {cuts}")
    _close(np.concatenate(got_other), want_other, dtype, f"{name} request decoding beside the portions")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small-2L", "xl-1L"])
def test_many_requests_decoding_together_with_page_reuse(real_dirs, real_plain, name, dtype):
    """(iii) 24 live requests bring single tokens for 8 steps after short prompts (one step of all
    the prompts, then 24-token steps: hundreds of (token, head) pairs, products of 17..64 rows).
    The pool holds exactly what is live: two requests end after three steps and two new ones
    take over their slots and pages."""
    from sandyrt_b200.engine.step import StepEntry

    rng = np.random.default_rng(5)
    lengths = [int(n) for n in rng.integers(5, 41, size=26)]
    decode = [8] * 26
    decode[3] = decode[11] = 3                     # these two end early ...
    lengths[3], lengths[11] = 20, 33
    lengths[24], lengths[25] = 15, 28              # ... and their successors grow to exactly their sizes
    seqs = [_ids(name, lengths[i] + decode[i], seed=100 + i) for i in range(26)]
    pages = lambda n: -(-n // 16)
    first = list(range(24))
    pool_pages = sum(pages(len(seqs[i])) for i in first)       # exactly what the first 24 hold at their ends
    eng = _engine(real_dirs[name], dtype, max_tokens=pool_pages * 16, max_requests=24)
    oracle = real_plain(name, STORE[dtype])
    got = {i: [] for i in range(26)}
    fed = {i: 0 for i in range(26)}

    def run(step_entries):
        entries = [StepEntry(i, seqs[i][fed[i]:fed[i] + n], [n - 1] if fed[i] + n >= lengths[i] else [])
                   for i, n in step_entries]
        out = eng.step(entries).cpu().numpy()
        r = 0
        for (i, n), e in zip(step_entries, entries):
            if e.want:
                got[i].append(out[r].copy())
                r += 1
            fed[i] += n
        for i, _ in step_entries:
            if fed[i] == len(seqs[i]):
                eng.release(i)
        eng.cache.alloc.check()

    run([(i, lengths[i]) for i in first])                           # all prompts in one step
    live = list(first)
    for step in range(8):
        if step == 3:                                               # the two that ended: their pages go to two new requests
            assert 3 not in eng.cache.alloc and 11 not in eng.cache.alloc
            run([(24, lengths[24]), (25, lengths[25])])
            live = [i for i in live if i not in (3, 11)] + [24, 25]
        live = [i for i in live if fed[i] < len(seqs[i])]
        run([(i, 1) for i in live])
    eng.check_status()
    assert eng.cache.alloc.pools[0].high_water == pool_pages
    for i in range(26):
        if fed[i] < len(seqs[i]):
            eng.release(i)
        n_rows = len(got[i])
        want = oracle.logits(seqs[i][:fed[i]], rows=list(range(lengths[i] - 1, lengths[i] - 1 + n_rows)))
        _close(np.stack(got[i]), want, dtype, f"{name} request {i} of 26")
    assert eng.cache.alloc.pools[0].free_pages == pool_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_requests", [1, 8])
def test_small_batches_decoding(real_dirs, real_plain, n_requests, dtype):
    """Decode steps of 1 and of 8 requests (the shapes the fused attention-block kernel takes in
    bfloat16: one block per token and head) over 40 single tokens each, after prompts of different
    lengths, so that contexts cross page edges at different steps."""
    from sandyrt_b200.engine.step import StepEntry

    name = "small-2L"
    eng = _engine(real_dirs[name], dtype, max_tokens=2048, max_requests=8)
    oracle = real_plain(name, STORE[dtype])
    lengths = [1, 15, 16, 17, 70, 129, 33, 250][:n_requests]
    seqs = [_ids(name, n + 40, seed=300 + i) for i, n in enumerate(lengths)]
    got = [[] for _ in seqs]
    out = eng.step([StepEntry(i, s[:lengths[i]], [lengths[i] - 1]) for i, s in enumerate(seqs)]).cpu().numpy()
    for i in range(n_requests):
        got[i].append(out[i].copy())
    for step in range(40):
        out = eng.step([StepEntry(i, [s[lengths[i] + step]], [0]) for i, s in enumerate(seqs)]).cpu().numpy()
        for i in range(n_requests):
            got[i].append(out[i].copy())
    eng.check_status()
    for i, s in enumerate(seqs):
        want = oracle.logits(s, rows=list(range(lengths[i] - 1, lengths[i] + 40)))
        _close(np.stack(got[i]), want, dtype, f"request {i} of {n_requests} decoding")
    eng.cache.alloc.check()


def test_greedy_generation_with_bursts_at_real_sizes(real_dirs, real_plain):
    """(iv) the entry point with bursts of decode steps, float32: the same tokens as the plain
    implementation's greedy loop."""
    from sandyrt_b200.engine.llm import LLM

    name = "small-2L"
    oracle = real_plain(name, "f32")
    prompts = [_ids(name, n, seed=200 + n) for n in (9, 70, 33, 130)]
    llm = LLM(real_dirs[name], dtype="float32", cache_tokens=2048, max_live=8, max_burst=8)
    got = llm.generate(prompts, max_tokens=12)
    assert llm.engine.graph_replays > 0
    for p, g in zip(prompts, got):
        want, reason = plain.generate_greedy(oracle, p, 12)
        assert g.output_ids == want and g.finish_reason == reason
    llm.engine.check_status()


def test_f16_checkpoint_is_widened_exactly_for_the_float32_path(tmp_path, real_plain):
    """A file that stores float16: the float32 path must compute with exactly those values (the
    plain implementation widens them to float32), not with a bfloat16 rounding of them."""
    from conftest import TINY, make_model_dir
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model

    d = make_model_dir(TINY["B"], str(tmp_path / "b_f16"), seed=77, store_dtype="float16")
    assert json.load(open(os.path.join(d, "config.json")))["n_embd"] == 96
    oracle = plain.PlainGPT2(d, store="f32")
    ids = np.random.default_rng(3).integers(0, 1000, size=60).tolist()
    model = load_model(d, device="cuda:0", dtype=torch.float32)
    eng = Engine(model, max_tokens=128, max_requests=2)
    got = eng.step([StepEntry("r", ids, list(range(60)))]).cpu().numpy()
    _close(got, oracle.logits(ids), "float32", "float16 file on the float32 path")
