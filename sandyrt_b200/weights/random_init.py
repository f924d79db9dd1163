"""Random-weights mode: write a model folder (config.json + model.safetensors) from a
configuration and a seed.

The reference has no such mode (its tests fill tensors by hand, make_pattern /
make_uniform_values, test/engine/CudaDeviceTest.cpp:302-312).  The distributions are:
matrix and table weights N(0, 0.02); biases N(0, 0.01); norm gains 1 + N(0, 0.02); norm
offsets N(0, 0.02).  Which of these a tensor gets is stated by the part that requests it
(TensorRequest.init).  Each tensor has its own generator seeded from (seed, tensor name),
so a tensor's values do not depend on which other tensors the model has.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict

import torch

from ..config.base import ModelConfig, save_config
from .loader import WEIGHT_FILE, TensorRequest
from .safetensors import write_safetensors

_INIT = {"weight": (0.0, 0.02), "bias": (0.0, 0.01), "gamma": (1.0, 0.02), "beta": (0.0, 0.02)}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(requests: Dict[str, TensorRequest], seed: int, dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    out = {}
    for name, req in requests.items():
        if req.integer or req.init == "zeros":
            out[name] = torch.zeros(req.shape, dtype=torch.int32 if req.integer else dtype)
            continue
        mean, std = _INIT[req.init]
        gen = torch.Generator(device="cpu")
        gen.manual_seed(_tensor_seed(seed, name))
        t = torch.randn(req.shape, generator=gen, dtype=torch.float32) * std + mean
        out[name] = t.to(torch.float32 if req.keep_32bit else dtype)
    return out


def write_random_model(config: ModelConfig, out_dir: str, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Create `out_dir` with config.json and a model.safetensors of seeded random weights
    stored in `dtype` (bfloat16 or float32).  Returns `out_dir`."""
    from ..models.model import build_model, describe

    config.validate()
    model = build_model(describe(config))
    tensors = random_tensors(model.tensor_requests(), seed, dtype)
    os.makedirs(out_dir, exist_ok=True)
    save_config(config, out_dir)
    write_safetensors(os.path.join(out_dir, WEIGHT_FILE), tensors)
    return out_dir
