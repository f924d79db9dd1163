"""The plain implementation itself (no GPU): anchored on the reference's CPU code through the
golden files of tests/golden/, plus checks of its parts."""
import importlib.util
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("case_name", ["tiny_a", "tiny_b_tanh"])
def test_plain_matches_the_reference_cpu_code(case_name, tmp_path):
    """tests/golden/<case>.json holds, per position, the five largest logits as the reference's
    cpu_runner printed them (%.6g).  The plain implementation must give the same ids and the
    same values to those six digits."""
    mg = _golden_module()
    with open(os.path.join(HERE, "golden", case_name + ".json")) as f:
        gold = json.load(f)
    case = mg.CASES[case_name]
    w = mg.golden_weights(case)
    ids = w.pop("__ids__").tolist()
    assert ids == gold["ids"]
    d = tmp_path / case_name
    d.mkdir()
    cfg = {k: v for k, v in case.items() if k not in ("seed", "n_tokens")}
    cfg["architectures"] = ["GPT2LMHeadModel"]
    (d / "config.json").write_text(json.dumps(cfg))
    mg.write_safetensors(str(d / "model.safetensors"), w)
    logits = plain.PlainGPT2(str(d)).logits(ids)
    for pos, top in enumerate(gold["top5"]):
        order = np.argsort(-logits[pos], kind="stable")[:5]
        assert [int(i) for i in order] == [t[0] for t in top], f"position {pos}: other top-5 ids"
        for (tid, val) in top:
            got = float(logits[pos, tid])
            assert got == pytest.approx(val, rel=2e-5, abs=2e-6), f"position {pos} id {tid}: {got} vs {val}"


def test_round_bf16_is_round_to_nearest_even():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 1, 5000), rng.normal(0, 1e-3, 500), [0.0, -0.0, 1.0, 3.3895314e38]]).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(plain.round_bf16(x), want)
    # exact ties go to the even mantissa
    tie = np.array([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8], dtype=np.float32)
    np.testing.assert_array_equal(plain.round_bf16(tie), np.array([1.0, 1.0 + 2 ** -6], dtype=np.float32))


def test_parts_against_closed_forms():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 2, size=(4, 10)).astype(np.float32)
    y = plain.layer_norm(x, np.ones(10, np.float32), np.zeros(10, np.float32), 1e-5)
    np.testing.assert_allclose(y.mean(-1), 0, atol=1e-6)
    np.testing.assert_allclose(y.var(-1), 1, atol=1e-4)
    u = np.array([-3.0, -1.0, 0.0, 0.5, 2.0], np.float32)
    np.testing.assert_allclose(plain.gelu_erf(u), [0.5 * v * (1 + math.erf(v / math.sqrt(2))) for v in u], rtol=1e-6)
    np.testing.assert_allclose(plain.gelu_new(u), plain.gelu_erf(u), atol=5e-3)      # the tanh form is an approximation
    assert np.abs(plain.gelu_new(u) - plain.gelu_erf(u)).max() > 1e-5               # ... but not the same function
    # attention: one key -> its value; uniform scores -> the mean of the visible values
    q = np.zeros((1, 3, 4), np.float32)
    k = rng.normal(size=(1, 3, 4)).astype(np.float32)
    v = rng.normal(size=(1, 3, 4)).astype(np.float32)
    o = plain.causal_attention(q, k, v, 0.5)
    np.testing.assert_allclose(o[0, 0], v[0, 0], atol=1e-6)
    np.testing.assert_allclose(o[0, 2], v[0].mean(0), atol=1e-6)
    np.testing.assert_allclose(plain.causal_attention(q, k, v, 0.5, window=2)[0, 2], v[0, 1:].mean(0), atol=1e-6)
    with pytest.raises(ValueError, match="out of range"):
        plain.embedding([0, 5], np.zeros((5, 2), np.float32))


def test_logits_at_a_position_do_not_depend_on_later_tokens(model_dirs):
    m = plain.PlainGPT2(model_dirs["B"])
    ids = np.random.default_rng(2).integers(0, 1000, size=30).tolist()
    full = m.logits(ids)
    np.testing.assert_allclose(m.logits(ids[:11])[-1], full[10], atol=1e-6)
    other = ids[:11] + [7] * 19
    np.testing.assert_allclose(m.logits(other)[:11], full[:11], atol=1e-6)


def test_plain_sampler_follows_the_reference_rules():
    l = np.array([0.1, 2.0, 2.0, -1.0, 1.5], np.float32)
    assert plain.sample_token(l) == 1                                   # ties: lower id (stable sort)
    assert plain.sample_token(l, temperature=1.0, top_k=1, u=0.99) == 1  # top_k = 1 is greedy
    draws = {plain.sample_token(l, temperature=1.0, top_k=2, u=u) for u in np.linspace(0, 0.999, 50)}
    assert draws == {1, 2}
    # top_p: shortest prefix whose share reaches top_p
    p = np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32))
    assert {plain.sample_token(p, 1.0, 0, 0.79, u) for u in np.linspace(0, 0.999, 50)} == {0, 1}
    assert {plain.sample_token(p, 1.0, 0, 0.81, u) for u in np.linspace(0, 0.999, 50)} == {0, 1, 2}
    with pytest.raises(ValueError, match="NaN"):
        plain.sample_token(np.array([0.0, np.nan], np.float32))
    # the distribution of draws follows softmax(l / T)
    us = (np.arange(20000) + 0.5) / 20000
    counts = np.bincount([plain.sample_token(l, 0.7, 0, 1.0, u) for u in us], minlength=5) / 20000
    want = np.exp(l / 0.7 - (l / 0.7).max()); want /= want.sum()
    np.testing.assert_allclose(counts, want, atol=2e-3)


def test_generate_greedy_stops(model_dirs):
    m = plain.PlainGPT2(model_dirs["A"])
    out, reason = plain.generate_greedy(m, [1, 2, 3], 6)
    assert len(out) == 6 and reason == "length"
    out2, reason2 = plain.generate_greedy(m, [1, 2, 3], 6, stop_ids=[out[2]])
    assert reason2 == "stop" and out2 == out[:out.index(out[2]) + 1]
    assert plain.generate_greedy(m, [1], 0) == ([], "length")
