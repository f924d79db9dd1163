"""Engine against the plain implementation, under every way of cutting the work.

The same requests are run: whole in one step; most of the prompt in one step and the last
32 tokens one by one; in portions of changing size down to two tokens; and mixed with other
requests (up to four live) in a pool with so few pages that they are used again.  Every
logit row is compared with the plain implementation's, in float32 and in bfloat16.
"""
import numpy as np
import pytest
import torch

from conftest import TINY

pytestmark = pytest.mark.gpu

# Tolerances.  float32: the engine and the plain implementation differ only in the order of
# float additions.  bfloat16: both round the same tensors to bfloat16, but a sum that lands
# near a rounding boundary can round the other way; one flip is 2^-9 relative on a value
# of order 1, and the logits (|.| about 0.2 with these weights) see a few of them.
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=6e-3, rtol=2e-2)}
STORE = {"float32": "f32", "bfloat16": "bf16"}


def _engine(model_dir, dtype, max_tokens, page_size=16, poison=True):
    from sandyrt_b200.engine.step import Engine
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dir, device="cuda:0", dtype=getattr(torch, dtype))
    eng = Engine(model, max_tokens=max_tokens, page_size=page_size, max_requests=8)
    if poison:
        eng.cache.device_caches.poison()
    return eng


def _prompts(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, TINY[name]["vocab_size"], size=n).tolist() for n in lengths]


def _close(got, want, dtype, what):
    got = np.asarray(got, dtype=np.float32)
    tol = TOL[dtype]
    err = np.abs(got - want)
    bound = tol["atol"] + tol["rtol"] * np.abs(want)
    if not (err <= bound).all():
        bad = np.argwhere(err > bound)[0]
        raise AssertionError(f"{what}: first wrong logit at row {bad[0]} col {bad[1]}: "
                             f"got {got[tuple(bad)]}, want {want[tuple(bad)]}, max err {err.max():.3e}")


def _run_cuts(eng, rid, ids, cuts):
    """Feed `ids` of one request in portions `cuts`, wanting every row; returns [T, V]."""
    from sandyrt_b200.engine.step import StepEntry

    rows, pos = [], 0
    for n in cuts:
        out = eng.step([StepEntry(rid, ids[pos:pos + n], list(range(n)))])
        rows.append(out.cpu().numpy().copy())
        pos += n
    assert pos == len(ids)
    eng.release(rid)
    return np.concatenate(rows, axis=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts(model_dirs, plain_models, name, dtype):
    eng = _engine(model_dirs[name], dtype, max_tokens=256)
    plain = plain_models(name, STORE[dtype])
    for i, ids in enumerate(_prompts(name, [5, 17, 33, 100, 1], seed=3)):
        got = _run_cuts(eng, f"r{i}", ids, [len(ids)])
        _close(got, plain.logits(ids), dtype, f"tiny {name} whole prompt of {len(ids)}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_then_decode_one_by_one(model_dirs, plain_models, name, dtype):
    eng = _engine(model_dirs[name], dtype, max_tokens=128)
    plain = plain_models(name, STORE[dtype])
    for i, ids in enumerate(_prompts(name, [40, 97], seed=5)):
        cuts = [len(ids) - 32] + [1] * 32
        got = _run_cuts(eng, f"r{i}", ids, cuts)
        _close(got, plain.logits(ids), dtype, f"tiny {name} prefill+decode of {len(ids)}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size(model_dirs, plain_models, name, dtype):
    eng = _engine(model_dirs[name], dtype, max_tokens=128)
    plain = plain_models(name, STORE[dtype])
    ids = _prompts(name, [101], seed=7)[0]
    for cuts in ([24, 24, 24, 24, 5], [2, 3, 17, 16, 15, 31, 2, 13, 2], [16, 16, 32, 1, 1, 35], [64, 37]):
        assert sum(cuts) == len(ids)
        got = _run_cuts(eng, "r", ids, cuts)
        _close(got, plain.logits(ids), dtype, f"tiny {name} cuts {cuts}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_requests_with_page_reuse(model_dirs, plain_models, name, dtype):
    """Up to four live requests; portions of some beside decoded tokens of others; the pool
    holds 12 pages of 16 tokens, so pages freed by a finished request are used again by the
    next (the pages are poisoned with NaN first: a read of a stale or unwritten slot shows)."""
    from sandyrt_b200.engine.step import StepEntry

    eng = _engine(model_dirs[name], dtype, max_tokens=192, page_size=16)
    plain = plain_models(name, STORE[dtype])
    lengths = [37, 50, 21, 64, 45, 30, 58, 17]
    prompts = _prompts(name, lengths, seed=9)
    want_logits = [plain.logits(p) for p in prompts]
    rng = np.random.default_rng(1)
    fed = [0] * len(prompts)
    got = [[] for _ in prompts]
    live, nxt, used_pages = [], 0, set()
    steps = 0
    while nxt < len(prompts) or live:
        # admit while fewer than four are live and the pool surely has room for the whole request
        while nxt < len(prompts) and len(live) < 4:
            need = -(-lengths[nxt] // 16)
            held = sum(-(-lengths[r] // 16) for r in live)
            if held + need > 12:
                break
            live.append(nxt)
            nxt += 1
        entries = []
        for r in live:
            left = lengths[r] - fed[r]
            if left > 8 and rng.random() < 0.6:
                n = int(rng.integers(2, min(left, 19) + 1))     # a portion of a prompt
            else:
                n = 1                                            # one token, as in decoding
            entries.append(StepEntry(r, prompts[r][fed[r]:fed[r] + n], list(range(n))))
        if rng.random() < 0.3 and len(entries) > 1:
            entries.pop(int(rng.integers(0, len(entries))))      # a request sits a step out
        out = eng.step(entries).cpu().numpy()
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.rid].append(out[row:row + n].copy())
            row += n
            fed[e.rid] += n
            used_pages.update(p for p in eng.cache.alloc.block_list(e.rid, 0))
        for r in list(live):
            if fed[r] == lengths[r]:
                eng.release(r)
                live.remove(r)
        eng.cache.alloc.check()
        steps += 1
    assert eng.cache.alloc.pools[0].free_pages == 12
    total_pages_if_never_reused = sum(-(-n // 16) for n in lengths)
    assert total_pages_if_never_reused > 12          # so pages were used again
    for r, ids in enumerate(prompts):
        _close(np.concatenate(got[r], axis=0), want_logits[r], dtype, f"tiny {name} mixed request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_recorded_prompt_step_serves_other_divisions_of_its_tokens(model_dirs, plain_models, dtype):
    """A prompt step is recorded as a CUDA graph under a key of counts (tokens, requests, wanted
    rows, longest portion, block-table width) and replayed for any step with the same counts.
    Three steps with the same counts divide their 48 tokens differently among three requests
    and start at different places of them; the later ones are served by the recording, and every
    row must still be right: whatever a launch takes from the host's lists would be stale."""
    from sandyrt_b200.engine.step import StepEntry

    name = "B"
    eng = _engine(model_dirs[name], dtype, max_tokens=512, page_size=16)
    plain = plain_models(name, STORE[dtype])
    prompts = _prompts(name, [72, 72, 80], seed=13)
    want = [plain.logits(p) for p in prompts]
    fed = [0, 0, 0]
    got = [[], [], []]
    replays = []
    for division in ([16, 8, 24], [8, 16, 24], [24, 24, 0], [24, 16, 8], [0, 8, 24]):
        entries = [StepEntry(r, prompts[r][fed[r]:fed[r] + n], list(range(n)))
                   for r, n in enumerate(division) if n]
        before = eng.graph_replays
        out = eng.step(entries).cpu().numpy()
        replays.append(eng.graph_replays - before)
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.rid].append(out[row:row + n].copy())
            row += n
            fed[e.rid] += n
    eng.check_status()
    # steps 0, 1 and 3 share one key (48 tokens, 3 requests, longest 24): the second records, the
    # third sight replays; steps 2 and 4 have other counts
    assert replays[1] == 1 and replays[3] == 1
    for r in range(3):
        _close(np.concatenate(got[r], axis=0), want[r][:fed[r]], dtype, f"request {r} under a replayed prompt graph")
