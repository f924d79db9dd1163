"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest
import torch

from conftest import TINY
from plain_gpt2 import generate_greedy, kept_set_and_cdf

pytestmark = pytest.mark.gpu


def _prompts(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, TINY[name]["vocab_size"], size=n).tolist() for n in lengths]


def _llm(model_dir, dtype="float32", **kw):
    from sandyrt_b200.engine.llm import LLM

    kw.setdefault("cache_tokens", 2048)
    kw.setdefault("max_live", 8)
    return LLM(model_dir, dtype=dtype, **kw)


def test_greedy_tiny_a_matches_plain(model_dirs, plain_models):
    """tiny A: 3 prompts of 5/17/33 tokens, 16 greedy tokens each, float32."""
    llm = _llm(model_dirs["A"])
    prompts = _prompts("A", [5, 17, 33], seed=21)
    plain = plain_models("A", "f32")
    want = [generate_greedy(plain, p, 16) for p in prompts]
    got = llm.generate(prompts, max_tokens=16)
    for g, (w_ids, w_reason), p in zip(got, want, prompts):
        assert g.output_ids == w_ids and g.finish_reason == w_reason == "length"
        assert g.prompt_tokens == len(p) and g.completion_tokens == 16
        assert g.decode_tokens_per_second > 0 and g.prefill_tokens_per_second > 0


def test_greedy_bfloat16_follows_the_plain_bfloat16_model(model_dirs, plain_models):
    """bfloat16 may break a near-tie differently; wherever the plain bfloat16 model's top two
    logits are clearly apart, the engine must pick the same token."""
    llm = _llm(model_dirs["B"], dtype="bfloat16")
    plain = plain_models("B", "bf16")
    for p in _prompts("B", [9, 40], seed=22):
        out = llm.generate(p, max_tokens=12)[0].output_ids
        ids = list(p)
        for tok in out:
            l = plain.logits(ids)[-1]
            top2 = np.sort(l)[-2:]
            if top2[1] - top2[0] > 2e-2:
                assert tok == int(np.argmax(l))
            ids.append(tok)


def test_temperature_sampling_tiny_b_chunked_prefill(model_dirs, plain_models):
    """tiny B: prompts of 1/40/64/100 tokens, prompt portions of 24 tokens, 20 tokens each at
    temperature 0.8 with a fixed seed.  Every drawn token must be the one the plain model's
    distribution assigns to the request's uniform number for that step."""
    from sandyrt_b200.sampling.sampler import uniform_for

    llm = _llm(model_dirs["B"], prefill_chunk_tokens=24, max_step_tokens=64)
    plain = plain_models("B", "f32")
    prompts = _prompts("B", [1, 40, 64, 100], seed=23)
    res = llm.generate(prompts, max_tokens=20, temperature=0.8, seed=1234)
    again = _llm(model_dirs["B"], prefill_chunk_tokens=7, max_step_tokens=33).generate(
        prompts, max_tokens=20, temperature=0.8, seed=1234)
    for i, (p, r, r2) in enumerate(zip(prompts, res, again)):
        assert len(r.output_ids) == 20 and r.finish_reason == "length"
        assert r.output_ids == r2.output_ids          # same seed, other portion sizes: same tokens
        ids = list(p)
        for step, tok in enumerate(r.output_ids):
            kept, cdf = kept_set_and_cdf(plain.logits(ids)[-1], 0.8)
            u = uniform_for(1234 + i, step)
            j = int(np.where(kept == tok)[0][0])
            lo = cdf[j - 1] if j else 0.0
            assert lo - 1e-4 <= u <= cdf[j] + 1e-4, f"request {i} step {step}: token {tok} does not match u={u}"
            ids.append(tok)
    assert len({tuple(r.output_ids) for r in res}) == 4        # different seeds per request


def test_stop_tokens_and_zero_max_tokens(model_dirs, plain_models):
    llm = _llm(model_dirs["A"])
    plain = plain_models("A", "f32")
    p = _prompts("A", [12], seed=24)[0]
    free_run, _ = generate_greedy(plain, p, 10)
    stop = free_run[4]
    first = free_run.index(stop)
    r = llm.generate(p, max_tokens=10, stop_token_ids=[stop])[0]
    assert r.output_ids == free_run[:first + 1] and r.finish_reason == "stop"   # the stop token is part of the output
    r0 = llm.generate(p, max_tokens=0)[0]
    assert r0.output_ids == [] and r0.finish_reason == "length" and r0.completion_tokens == 0


def test_long_decoding_to_the_last_position(model_dirs, plain_models):
    """Decode until the model's positions run out (128 for tiny A): many pages, every position."""
    llm = _llm(model_dirs["A"])
    plain = plain_models("A", "f32")
    p = _prompts("A", [3], seed=25)[0]
    r = llm.generate(p, max_tokens=500)[0]
    want, reason = generate_greedy(plain, p, 500)
    assert r.finish_reason == reason == "length"
    assert len(p) + len(r.output_ids) == TINY["A"]["n_positions"] + 1 or len(r.output_ids) == len(want)
    n = min(len(want), len(r.output_ids))
    assert r.output_ids[:n] == want[:n] and n >= 120


def test_first_tokens_of_a_sequence(model_dirs, plain_models):
    """A prompt of a single token, and the very first logits of a sequence."""
    from sandyrt_b200.engine.step import StepEntry

    llm = _llm(model_dirs["B"])
    plain = plain_models("B", "f32")
    for tok in (0, 999, 417):
        out = llm.engine.step([StepEntry(f"one-{tok}", [tok], [0])]).cpu().numpy()
        llm.engine.release(f"one-{tok}")
        np.testing.assert_allclose(out[0], plain.logits([tok])[0], atol=2e-5, rtol=1e-4)
    r = llm.generate([417], max_tokens=5)[0]
    assert r.output_ids == generate_greedy(plain, [417], 5)[0]


def test_preemption_does_not_change_the_output(model_dirs):
    """With a cache too small for all requests at once some are preempted and recomputed; the
    tokens must be the same as with plenty of room."""
    prompts = _prompts("A", [30, 28, 26, 31], seed=26)
    roomy = _llm(model_dirs["A"], cache_tokens=4096).generate(prompts, max_tokens=40)
    tight_llm = _llm(model_dirs["A"], cache_tokens=160, page_size=16)     # 10 pages for 4 x ~70 tokens
    tight = tight_llm.generate(prompts, max_tokens=40)
    assert tight_llm.scheduler.stats["preemptions"] > 0
    assert [r.output_ids for r in tight] == [r.output_ids for r in roomy]
    assert sum(r.preemptions for r in tight) == tight_llm.scheduler.stats["preemptions"]
    tight_llm.engine.cache.alloc.check()
    assert tight_llm.engine.cache.alloc.free_pages() == 10


def test_refusals_through_the_entry_point(model_dirs):
    from sandyrt_b200.engine.scheduler import RequestRefused

    llm = _llm(model_dirs["A"])
    with pytest.raises(RequestRefused, match="empty"):
        llm.generate([[]], max_tokens=4)
    with pytest.raises(RequestRefused, match="vocabulary"):
        llm.generate([5, 512], max_tokens=4)
    with pytest.raises(RequestRefused, match="positions"):
        llm.generate(list(range(129)), max_tokens=4)
    with pytest.raises(ValueError, match="top_p"):
        llm.generate([1, 2], max_tokens=4, top_p=0.0)


def test_on_token_callback_can_cancel(model_dirs):
    llm = _llm(model_dirs["A"])
    seen = []

    def cb(index, token):
        seen.append((index, token))
        return len(seen) < 3

    r = llm.generate([5, 6, 7], max_tokens=50, on_token=cb)[0]
    assert r.finish_reason == "cancelled" and len(r.output_ids) == 3 == len(seen)
    assert llm.engine.cache.alloc.free_slots() == 8      # everything was given back


def test_bursts_give_the_same_tokens_as_single_steps(model_dirs):
    """Several decode steps per look of the host (tokens fed back on the device) against one
    step per look: same tokens, same finish reasons, also when a request stops part of the way
    through a burst and when pages are tight."""
    prompts = _prompts("B", [3, 40, 17, 64], seed=31)
    for kw in (dict(max_tokens=37), dict(max_tokens=45, temperature=0.9, seed=5), dict(max_tokens=30, temperature=0.7, top_k=20, top_p=0.9, seed=9)):
        single = _llm(model_dirs["B"], max_burst=1).generate(prompts, **kw)
        burst_llm = _llm(model_dirs["B"], max_burst=8)
        burst = burst_llm.generate(prompts, **kw)
        assert [r.output_ids for r in burst] == [r.output_ids for r in single]
        assert [r.finish_reason for r in burst] == [r.finish_reason for r in single]
        assert burst_llm.engine.graph_replays > 0
    # a stop token in the middle of a burst: the tokens after it are dropped
    free = _llm(model_dirs["B"], max_burst=1).generate(prompts[1], max_tokens=40)[0].output_ids
    stop = free[13]
    cut = free.index(stop)
    r = _llm(model_dirs["B"], max_burst=8).generate(prompts[1], max_tokens=40, stop_token_ids=[stop])[0]
    assert r.output_ids == free[:cut + 1] and r.finish_reason == "stop"
    # tight pages: bursts shrink instead of failing, preemption still works
    tight = _llm(model_dirs["B"], cache_tokens=224, page_size=16, max_burst=8)
    roomy = _llm(model_dirs["B"], cache_tokens=4096, max_burst=1)
    kw = dict(max_tokens=50)
    assert [r.output_ids for r in tight.generate(prompts, **kw)] == [r.output_ids for r in roomy.generate(prompts, **kw)]
    tight.engine.cache.alloc.check()


def test_bursts_queued_ahead_give_the_same_tokens(model_dirs):
    """The next burst is queued before the last one's tokens are read: same tokens as without,
    when requests of one batch stop at different times (stop tokens, different limits), when
    another request arrives in the middle, and two generate calls in a row on one engine."""
    prompts = _prompts("B", [3, 40, 17, 64], seed=31)
    for kw in (dict(max_tokens=61), dict(max_tokens=50, temperature=0.9, seed=5)):
        plain = _llm(model_dirs["B"], pipeline_bursts=False)
        ahead = _llm(model_dirs["B"], pipeline_bursts=True)
        a, b = plain.generate(prompts, **kw), ahead.generate(prompts, **kw)
        assert [r.output_ids for r in a] == [r.output_ids for r in b]
        assert ahead.bursts_queued_ahead > 0 and plain.bursts_queued_ahead == 0
        # a stop token that ends one request in the middle of a burst while a later burst is queued
        stop = a[1].output_ids[20]
        a2 = plain.generate(prompts, stop_token_ids=[stop], **kw)
        b2 = ahead.generate(prompts, stop_token_ids=[stop], **kw)
        assert [r.output_ids for r in a2] == [r.output_ids for r in b2]
        assert [r.finish_reason for r in a2] == [r.finish_reason for r in b2]
        assert any(r.finish_reason == "stop" for r in b2)
        ahead.engine.cache.alloc.check()
        ahead.engine.check_status()
    # a request added while bursts are in flight joins after they have drained
    llm = _llm(model_dirs["B"], pipeline_bursts=True)
    first = llm.add_request(prompts[1], max_tokens=60)
    for _ in range(3):
        llm.step()
    second = llm.add_request(prompts[2], max_tokens=20)
    while llm.has_work():
        llm.step()
    ref = _llm(model_dirs["B"], max_burst=1)
    assert llm.result(first).output_ids == ref.generate(prompts[1], max_tokens=60)[0].output_ids
    assert llm.result(second).output_ids == ref.generate(prompts[2], max_tokens=20)[0].output_ids
    llm.engine.cache.alloc.check()


def test_a_recorded_burst_serves_a_batch_whose_member_was_replaced(model_dirs):
    """A whole burst of decode steps is recorded as one graph once its shape has come by three
    times.  Here three requests decode together long enough for that; then one of them ends and
    a waiting request of another length takes its place, so the same burst shape comes by again
    with another member at another position.  The tokens must equal those of single steps."""
    prompts = _prompts("B", [21, 34, 9, 50], seed=41)
    limits = [120, 120, 65, 40]

    def run(max_burst):
        llm = _llm(model_dirs["B"], max_live=3, max_burst=max_burst)
        rids = [llm.add_request(p, max_tokens=m) for p, m in zip(prompts[:3], limits[:3])]
        while llm.has_work():
            llm.step()
            if len(rids) == 3 and llm.finished(rids[2]):       # the third has ended: the fourth takes its place
                rids.append(llm.add_request(prompts[3], max_tokens=limits[3]))
        return llm, [llm.result(r).output_ids for r in rids]

    single, want = run(1)
    burst, got = run(8)
    assert got == want
    assert [len(g) for g in got] == limits
    assert burst.engine.burst_graphs_recorded > 0, "no whole-burst graph was recorded"
    burst.engine.check_status()
    burst.engine.cache.alloc.check()
