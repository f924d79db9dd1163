"""Random-weights mode: write a model folder (config.json + model.safetensors) from a
configuration and a seed.

The reference has no such mode (its tests fill tensors by hand, make_pattern / make_uniform_values,
test/engine/CudaDeviceTest.cpp:302-312).  The distributions are: matrix and table weights
N(0, 0.02); biases N(0, 0.01); norm gains 1 + N(0, 0.02); norm offsets N(0, 0.02).  Which of these
a tensor gets is stated by the part that requests it (TensorRequest.init).  Each tensor has its own
counter-based generator keyed by (seed, tensor name), so a tensor's values do not depend on which
other tensors the model has.  The generator is the host library's (core/weights.cpp).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import core
from ..config.base import ModelConfig
from .loader import TensorRequest, requests_to_json
from .safetensors import tensor_at

_STORE = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16"}


def random_tensors(requests: Dict[str, TensorRequest], seed: int, dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    out = core.call("global", None, "random_tensors", requests=requests_to_json(requests), seed=int(seed), dtype=_STORE[dtype])
    handle = core.Handle("weights", out["handle"])
    return {name: tensor_at(entry, handle) for name, entry in out["tensors"].items()}


def write_random_model(config: ModelConfig, out_dir: str, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> str:
    """Create `out_dir` with config.json and a model.safetensors of seeded random weights stored
    in `dtype` (bfloat16, float16 or float32).  Returns `out_dir`."""
    return core.call("global", None, "write_random_model", config=config.to_dict(), out_dir=out_dir, seed=int(seed),
                     dtype=_STORE[dtype])
