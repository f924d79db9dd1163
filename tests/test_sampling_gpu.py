"""The device sampler against the plain sampler: greedy ties, temperature, top-k, top-p."""
import numpy as np
import pytest
import torch

from plain_gpt2 import kept_set_and_cdf, sample_token

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sample(logits, temperature=None, top_k=None, top_p=None, uniform=None):
    from sandyrt_b200.csrc import ops

    n = logits.shape[0]
    out = torch.full((n,), -7, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    f = lambda v, dt: None if v is None else torch.tensor(v, dtype=dt, device=DEV)
    ops.sample(logits, out, temperature=f(temperature, torch.float32), top_k=f(top_k, torch.int32),
               top_p=f(top_p, torch.float32), uniform=f(uniform, torch.float32), status=status)
    return out.cpu().tolist(), int(status.item())


@pytest.mark.parametrize("vocab", [512, 1000, 50257, 37])
def test_greedy_is_first_maximum(vocab):
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(6, vocab, generator=g)
    logits[1, [5, vocab - 1, 9]] = 9.0                 # a tie: the lowest id wins (stable sort, Sampler.cpp:69-74)
    logits[2, vocab - 1] = 11.0                        # the last id
    logits[3] = -float("inf")                          # nothing finite: still the first
    logits[4, 3] = float("inf")
    got, status = _sample(logits.to(DEV))
    want = [sample_token(logits[i].numpy()) for i in range(6)]
    assert got == want and status == 0
    assert got[1] == 5 and got[2] == vocab - 1 and got[3] == 0 and got[4] == 3


def test_nan_is_reported():
    logits = torch.zeros(2, 100)
    logits[1, 7] = float("nan")
    got, status = _sample(logits.to(DEV))
    assert got[0] == 0 and got[1] == -1 and status & 1


def _check_draws(logits, temperature, top_k, top_p, uniforms):
    """Every device draw must be the id whose CDF interval holds u (up to float rounding at the
    interval's edges), and must lie in the kept set of the plain sampler."""
    n = logits.shape[0]
    got, status = _sample(logits.to(DEV), temperature, top_k, top_p, uniforms)
    assert status == 0
    for i in range(n):
        l = logits[i].numpy()
        if temperature[i] == 0.0:
            assert got[i] == sample_token(l)
            continue
        ids, cdf = kept_set_and_cdf(l, temperature[i], top_k[i], top_p[i])
        assert got[i] in ids, f"row {i}: id {got[i]} is outside the kept set of {len(ids)}"
        j = int(np.where(ids == got[i])[0][0])
        lo = cdf[j - 1] if j > 0 else 0.0
        hi = cdf[j]
        assert lo - 1e-4 <= uniforms[i] <= hi + 1e-4, f"row {i}: u={uniforms[i]} not in [{lo}, {hi}]"


@pytest.mark.parametrize("vocab", [1000, 50257])
def test_temperature_top_k_top_p(vocab):
    rng = np.random.default_rng(vocab)
    n = 64
    logits = torch.from_numpy(rng.normal(0, 2.0, size=(n, vocab)).astype(np.float32))
    logits[:, 17] += 3.0
    temperature = [float(t) for t in rng.choice([0.0, 0.3, 0.8, 1.0, 1.7], size=n)]
    top_k = [int(k) for k in rng.choice([0, 1, 2, 10, 50, vocab, vocab + 5], size=n)]
    top_p = [float(p) for p in rng.choice([1.0, 0.95, 0.5, 0.1, 1e-6], size=n)]
    uniforms = [float(u) for u in rng.random(n).astype(np.float32)]
    uniforms[0], uniforms[1] = 0.0, float(np.float32(1.0 - 2 ** -24))
    _check_draws(logits, temperature, top_k, top_p, uniforms)


def test_ties_at_the_top_k_cut_go_to_the_lower_ids():
    logits = torch.full((1, 200), -5.0)
    logits[0, [10, 20, 30, 40, 50]] = 2.0               # five tied candidates, top_k = 3 keeps ids 10, 20, 30
    seen = set()
    for u in np.linspace(0.0, 0.999, 41):
        got, _ = _sample(logits.to(DEV), [1.0], [3], [1.0], [float(u)])
        seen.add(got[0])
    assert seen == {10, 20, 30}


def test_top_p_keeps_the_shortest_prefix():
    # probabilities 0.5, 0.3, 0.15, 0.05 at ids 3, 1, 7, 5
    p = np.array([0.5, 0.3, 0.15, 0.05])
    logits = torch.full((1, 16), -1e4)
    for idx, prob in zip([3, 1, 7, 5], p):
        logits[0, idx] = float(np.log(prob))
    for top_p, allowed in ((0.4, {3}), (0.5, {3}), (0.51, {3, 1}), (0.8, {3, 1}), (0.81, {3, 1, 7}), (1.0, {3, 1, 7, 5})):
        seen = set()
        for u in np.linspace(0.0, 0.9999, 101):
            got, _ = _sample(logits.to(DEV), [1.0], [0], [top_p], [float(u)])
            seen.add(got[0])
        assert seen == allowed, (top_p, seen)


def test_uniform_numbers_are_counter_based():
    from sandyrt_b200.sampling.sampler import uniform_for

    a = [uniform_for(42, i) for i in range(1000)]
    assert a == [uniform_for(42, i) for i in range(1000)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert abs(np.mean(a) - 0.5) < 0.05 and len(set(a)) > 990
    assert a[:5] != [uniform_for(43, i) for i in range(5)]
