"""Weight files: container errors and the one binding error that lists everything (no GPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, make_model_dir


def _requests(model_dir):
    from sandyrt_b200.config.base import load_config
    from sandyrt_b200.models.model import build_model, describe

    spec = describe(load_config(model_dir))
    return build_model(spec).tensor_requests(), spec


def _rewrite(model_dir, edit):
    from sandyrt_b200.weights.safetensors import SafetensorsFile, write_safetensors

    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    edit(tensors)
    write_safetensors(path, tensors)


def test_roundtrip_and_dtypes(tmp_path):
    from sandyrt_b200.weights.loader import load_weights

    d = make_model_dir(TINY_A, str(tmp_path / "m32"), seed=1, store_dtype="float32")
    req, spec = _requests(d)
    t = load_weights(d, req, spec.name_prefixes, spec.ignored_tensors)
    assert set(t) == set(req)
    assert t["wte.weight"].dtype == torch.float32          # stored in 32-bit stays so
    d16 = make_model_dir(TINY_A, str(tmp_path / "m16"), seed=1, store_dtype="bfloat16")
    t16 = load_weights(d16, req, spec.name_prefixes, spec.ignored_tensors)
    assert t16["wte.weight"].dtype == torch.bfloat16
    # same seed, same values up to the storage rounding
    assert torch.equal(t["h.0.ln_1.weight"].to(torch.bfloat16), t16["h.0.ln_1.weight"])
    # gains are about 1, everything else about 0
    assert abs(float(t["h.1.ln_2.weight"].mean()) - 1.0) < 0.05
    assert abs(float(t["h.1.attn.c_attn.weight"].std()) - 0.02) < 0.005
    assert abs(float(t["h.1.attn.c_attn.bias"].std()) - 0.01) < 0.005


def test_seed_changes_values_and_names_fix_them(tmp_path):
    from sandyrt_b200.weights.safetensors import SafetensorsFile

    a = SafetensorsFile(os.path.join(make_model_dir(TINY_A, str(tmp_path / "a"), seed=1), "model.safetensors"))
    b = SafetensorsFile(os.path.join(make_model_dir(TINY_A, str(tmp_path / "b"), seed=1), "model.safetensors"))
    c = SafetensorsFile(os.path.join(make_model_dir(TINY_A, str(tmp_path / "c"), seed=2), "model.safetensors"))
    assert torch.equal(a.tensor("wpe.weight"), b.tensor("wpe.weight"))
    assert not torch.equal(a.tensor("wpe.weight"), c.tensor("wpe.weight"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from sandyrt_b200.weights.loader import WeightBindingError, load_weights

    d = make_model_dir(TINY_A, str(tmp_path / "m"), seed=1)

    def edit(t):
        del t["h.0.ln_1.bias"]
        del t["h.1.mlp.c_fc.weight"]
        t["h.7.extra.weight"] = torch.zeros(3)
        t["wpe.weight"] = torch.zeros(100, 64)
        t["h.0.attn.c_proj.weight"] = torch.zeros(64, 32)
    _rewrite(d, edit)
    req, spec = _requests(d)
    with pytest.raises(WeightBindingError) as ei:
        load_weights(d, req, spec.name_prefixes, spec.ignored_tensors)
    e = ei.value
    assert e.missing == ["h.0.ln_1.bias", "h.1.mlp.c_fc.weight"]
    assert e.unexpected == ["h.7.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["h.0.attn.c_proj.weight", "wpe.weight"]
    msg = str(e)
    for word in ("h.0.ln_1.bias", "h.7.extra.weight", "wpe.weight is [100, 64], expected [128, 64]"):
        assert word in msg


def test_prefix_and_ignored_buffers(tmp_path):
    from sandyrt_b200.weights.loader import load_weights

    d = make_model_dir(TINY_A, str(tmp_path / "m"), seed=1)

    def edit(t):
        for k in list(t):
            t["transformer." + k] = t.pop(k)
        t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)       # stored causal mask
        t["lm_head.weight"] = t["transformer.wte.weight"].clone()     # stored copy of the tied table
    _rewrite(d, edit)
    req, spec = _requests(d)
    t = load_weights(d, req, spec.name_prefixes, spec.ignored_tensors)
    assert t["wte.weight"].shape == (512, 64)


def test_integer_where_floats_are_wanted(tmp_path):
    from sandyrt_b200.weights.loader import WeightBindingError, load_weights

    d = make_model_dir(TINY_A, str(tmp_path / "m"), seed=1)
    _rewrite(d, lambda t: t.__setitem__("ln_f.bias", torch.zeros(64, dtype=torch.int64)))
    req, spec = _requests(d)
    with pytest.raises(WeightBindingError, match="ln_f.bias is int64"):
        load_weights(d, req, spec.name_prefixes, spec.ignored_tensors)


@pytest.mark.parametrize("damage,word", [
    (lambda b: b[:5], "too short"),
    (lambda b: struct.pack("<Q", 1 << 40) + b[8:], "header length"),
    (lambda b: b[:8] + b"{" * (struct.unpack("<Q", b[:8])[0]) + b[8 + struct.unpack("<Q", b[:8])[0]:], "JSON"),
    (lambda b: b[:-100], "outside the payload"),
])
def test_container_faults_are_errors_not_crashes(tmp_path, damage, word):
    from sandyrt_b200.weights.safetensors import SafetensorsFile, WeightFileError

    d = make_model_dir(TINY_A, str(tmp_path / "m"), seed=1)
    path = os.path.join(d, "model.safetensors")
    blob = open(path, "rb").read()
    open(path, "wb").write(damage(blob))
    with pytest.raises(WeightFileError, match=word):
        SafetensorsFile(path)


def test_missing_file_and_unknown_dtype(tmp_path):
    from sandyrt_b200.weights.safetensors import SafetensorsFile, WeightFileError

    with pytest.raises(WeightFileError, match="not found"):
        SafetensorsFile(str(tmp_path / "nope.safetensors"))
    head = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}).encode()
    p = tmp_path / "odd.safetensors"
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0\0")
    with pytest.raises(WeightFileError, match="unsupported dtype F8_E4M3"):
        SafetensorsFile(str(p))


def test_overlapping_tensors_are_refused(tmp_path):
    from sandyrt_b200.weights.safetensors import SafetensorsFile, WeightFileError

    head = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                       "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    p = tmp_path / "overlap.safetensors"
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 12)
    with pytest.raises(WeightFileError, match="overlap"):
        SafetensorsFile(str(p))
