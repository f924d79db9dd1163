"""Shared fixtures: two tiny GPT-2 configurations that differ in every size and option,
written as model folders with seeded random weights into a temporary directory."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


# tiny A: 2 layers, width 64, 4 heads of 16, inner 256 (4x), vocab 512, 128 positions,
#         eps 1e-5, gelu_new, no per-layer attention scaling
TINY_A = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=64, n_head=4,
              n_inner=256, vocab_size=512, n_positions=128, layer_norm_epsilon=1e-5,
              activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
              tie_word_embeddings=True)
# tiny B: 3 layers, width 96, 3 heads of 32, inner 320 (not 4x), vocab 1000 (no power of two),
#         256 positions, eps 1e-6, exact gelu, attention scaled by 1/(layer+1)
TINY_B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=3, n_embd=96, n_head=3,
              n_inner=320, vocab_size=1000, n_positions=256, layer_norm_epsilon=1e-6,
              activation_function="gelu", scale_attn_by_inverse_layer_idx=True,
              tie_word_embeddings=True)
# tiny C: odd sizes for the kernels: 5 heads of 48, width 240, inner 200, vocab 777
TINY_C = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=240, n_head=5,
              n_inner=200, vocab_size=777, n_positions=320, layer_norm_epsilon=3e-5,
              activation_function="gelu_new", scale_attn_by_inverse_layer_idx=True,
              tie_word_embeddings=True)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_model_dir(raw_config: dict, path: str, seed: int, store_dtype: str = "float32") -> str:
    import torch

    from sandyrt_b200.config.gpt2 import GPT2Config
    from sandyrt_b200.weights.random_init import write_random_model

    cfg = GPT2Config.from_dict(raw_config)
    write_random_model(cfg, path, seed=seed, dtype=getattr(torch, store_dtype))
    return path


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{"A": dir, "B": dir, "C": dir}: folders with config.json + model.safetensors (float32)."""
    base = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(raw, str(base / f"tiny_{name}"), seed=11 + i)
            for i, (name, raw) in enumerate(TINY.items())}


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    from plain_gpt2 import PlainGPT2

    cache = {}

    def get(name: str, store: str):
        key = (name, store)
        if key not in cache:
            cache[key] = PlainGPT2(model_dirs[name], store=store)
        return cache[key]

    return get
