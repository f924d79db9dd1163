"""Typed configuration and the architecture registry (no GPU)."""
import json
import os

import pytest

from conftest import TINY_A, TINY_B


def test_gpt2_config_reads_its_own_keys():
    from sandyrt_b200.config.gpt2 import GPT2Config

    a = GPT2Config.from_dict(TINY_A)
    b = GPT2Config.from_dict(TINY_B)
    a.validate(); b.validate()
    assert (a.n_layer, a.n_embd, a.n_head, a.head_dim, a.inner_dim, a.vocab_size, a.n_positions) == \
        (2, 64, 4, 16, 256, 512, 128)
    assert (b.n_layer, b.n_embd, b.n_head, b.head_dim, b.inner_dim, b.vocab_size, b.n_positions) == \
        (3, 96, 3, 32, 320, 1000, 256)
    assert a.layer_norm_epsilon == 1e-5 and b.layer_norm_epsilon == 1e-6
    assert a.activation_function == "gelu_new" and b.activation_function == "gelu"
    assert not a.scale_attn_by_inverse_layer_idx and b.scale_attn_by_inverse_layer_idx


def test_defaults_of_absent_keys():
    from sandyrt_b200.config.gpt2 import GPT2Config

    raw = dict(architectures=["GPT2LMHeadModel"], n_layer=1, n_embd=32, n_head=2, n_ctx=64, vocab_size=100)
    c = GPT2Config.from_dict(raw)
    c.validate()
    assert c.n_positions == 64            # legacy n_ctx
    assert c.inner_dim == 128             # n_inner null -> 4 * n_embd
    assert c.tie_word_embeddings and c.scale_attn_weights and not c.scale_attn_by_inverse_layer_idx


@pytest.mark.parametrize("patch,word", [
    ({"n_head": 5}, "divisible"),
    ({"activation_function": "relu"}, "activation_function"),
    ({"n_layer": 0}, "n_layer"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"eos_token_id": 99999}, "eos_token_id"),
])
def test_bad_configs_are_refused(patch, word):
    from sandyrt_b200.config.base import ConfigError
    from sandyrt_b200.config.gpt2 import GPT2Config

    raw = dict(TINY_A); raw.update(patch)
    with pytest.raises(ConfigError, match=word):
        GPT2Config.from_dict(raw).validate()


def test_missing_key_is_named():
    from sandyrt_b200.config.base import ConfigError
    from sandyrt_b200.config.gpt2 import GPT2Config

    raw = dict(TINY_A); del raw["n_embd"]
    with pytest.raises(ConfigError, match="n_embd"):
        GPT2Config.from_dict(raw)


def test_registry_chooses_the_class_by_config_json(tmp_path):
    from sandyrt_b200.config.base import ConfigError, load_config
    from sandyrt_b200.config.gpt2 import GPT2Config
    from sandyrt_b200.registry import architectures

    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, GPT2Config) and cfg.n_inner == 320
    assert "GPT2LMHeadModel" in architectures()
    raw = dict(TINY_B); raw["architectures"] = ["NoSuchModel"]
    (tmp_path / "config.json").write_text(json.dumps(raw))
    with pytest.raises(ConfigError, match="NoSuchModel.*GPT2LMHeadModel"):
        load_config(str(tmp_path))
    os.remove(tmp_path / "config.json")
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))


def test_model_description_is_data(model_dirs):
    """Layer kinds, sizes, run order and tensor names all come out of describe(config)."""
    from sandyrt_b200.config.base import load_config
    from sandyrt_b200.models.model import build_model, describe

    cfg = load_config(model_dirs["B"])
    spec = describe(cfg)
    assert len(spec.layers) == 3 and [c.layer for c in spec.schedule] == [0, 1, 2]
    assert spec.layers[2].mixer.params["scale"] == pytest.approx(1 / (32 ** 0.5) / 3)
    assert spec.layers[1].feed_forward.params["inner"] == 320
    model = build_model(spec)
    req = model.tensor_requests()
    assert req["h.1.attn.c_attn.weight"].shape == (96, 288)
    assert req["h.2.mlp.c_proj.weight"].shape == (320, 96)
    assert req["wte.weight"].shape == (1000, 96) and req["wpe.weight"].shape == (256, 96)
    assert "lm_head.weight" not in req      # tied


def test_a_model_an_llm_has_taken_over_cannot_be_handed_to_a_second_engine():
    """LLM() takes its model over; passing the same Model object again raises (it used to crash)."""
    import sandyrt_b200.core as core
    from sandyrt_b200.models.model import Model

    m = Model.__new__(Model)
    m._h = core.Handle("llm", 0, owned=False)
    with pytest.raises(ValueError, match="already belongs"):
        m._handle_for_engine()
    m._h = core.Handle("model", 1234, owned=False)
    assert m._handle_for_engine() == 1234
