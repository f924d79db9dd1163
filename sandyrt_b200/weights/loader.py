"""Binding of weight-file tensors to a model's parts, by name.

The reference resolves `weight("h.3.attn.c_proj.weight")` against the file's descriptors and fails
on the first name it cannot find ("weight not found: <name>", src/ir/MidIRMaterializer.cpp:186-194;
"missing weight buffer", src/engine/Engine.cpp:1143-1147).  Here the model states every tensor it
wants with its shape up front, the file is checked against that list in one pass, and ONE
WeightBindingError lists everything that is wrong: missing tensors, unexpected tensors, and tensors
of the wrong shape or kind.  The check is the host library's (core/weights.cpp); `load_weights`
returns what it bound as torch views, for callers that want to look at the values.

Storage dtypes on the host after loading: floating-point tensors stay as the file stores them
(BF16, F16 or F32: views of the mapping, nothing is rounded here); the parts convert what feeds
their matrix products to the engine's compute dtype when they bind, so each value is rounded at
most once: an F16 file is widened exactly for the float32 path and rounded to bfloat16 for the
bfloat16 path.  A part may ask that a tensor stored in 32-bit stays so (`keep_32bit`).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Sequence, Tuple

import torch

from .. import core
from ..errors import WeightBindingError, WeightFileError  # noqa: F401  (re-exported)
from .safetensors import tensor_at

WEIGHT_FILE = "model.safetensors"


@dataclasses.dataclass(frozen=True)
class TensorRequest:
    """What a part expects of one tensor of the weight file."""
    shape: Tuple[int, ...]
    integer: bool = False      # an integer table (kept as int32) rather than floats
    keep_32bit: bool = False   # if stored as F32, stay F32 whatever the compute dtype
    # How the random-weights mode fills it: "weight" N(0, 0.02), "bias" N(0, 0.01),
    # "gamma" 1 + N(0, 0.02), "beta" N(0, 0.02), "zeros".
    init: str = "weight"


def requests_to_json(requests: Dict[str, TensorRequest]) -> Dict[str, dict]:
    return {n: {"shape": list(r.shape), "integer": r.integer, "keep_32bit": r.keep_32bit, "init": r.init}
            for n, r in requests.items()}


def requests_from_json(j: Dict[str, dict]) -> Dict[str, TensorRequest]:
    return {n: TensorRequest(tuple(r["shape"]), r.get("integer", False), r.get("keep_32bit", False), r.get("init", "weight"))
            for n, r in j.items()}


def load_weights(model_dir: str, requests: Dict[str, TensorRequest], prefixes: Sequence[str] = ("",),
                 ignored: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Open `model_dir/model.safetensors`, check it against `requests` and return the requested
    tensors by their un-prefixed names (host tensors, views of the mapping)."""
    out = core.call("global", None, "load_weights", model_dir=model_dir, requests=requests_to_json(requests),
                    prefixes=list(prefixes), ignored=list(ignored))
    handle = core.Handle("weights", out["handle"])
    return {name: tensor_at(entry, handle) for name, entry in out["tensors"].items()}
