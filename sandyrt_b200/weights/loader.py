"""Binding of weight-file tensors to a model's parts, by name.

The reference resolves `weight("h.3.attn.c_proj.weight")` against the file's descriptors
and fails on the first name it cannot find ("weight not found: <name>",
src/ir/MidIRMaterializer.cpp:186-194; "missing weight buffer", src/engine/Engine.cpp:1143-1147).
Here the model states every tensor it wants with its shape up front, the file is checked
against that list in one pass, and ONE WeightBindingError lists everything that is wrong:
missing tensors, unexpected tensors, and tensors of the wrong shape.

Storage dtypes on the host after loading: floating-point tensors stay as the file stores them
(BF16, F16 or F32: views of the mapping, nothing is rounded here); I32/I64/U8/BOOL tables ->
int32.  The parts cast what feeds their matrix products to the engine's compute dtype when
they bind, so each value is rounded at most once: an F16 file is widened exactly for the
float32 path and rounded to bfloat16 for the bfloat16 path.  A part may ask that a tensor
stored in 32-bit stays so (`keep_32bit`).
"""
from __future__ import annotations

import dataclasses
import os
import re
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors import SafetensorsFile, WeightFileError

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


class WeightBindingError(Exception):
    """The weight file does not hold exactly the tensors the model needs."""

    def __init__(self, path: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_kind: List[Tuple[str, str]] = ()):
        self.path = path
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = [f"{path}: weight file does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong dtypes ({len(self.wrong_kind)}): " + ", ".join(
                f"{n} is {got}" for n, got in self.wrong_kind))
        super().__init__("\n".join(lines))


def _detect_prefix(names: Iterable[str], wanted: Iterable[str], prefixes: Sequence[str]) -> str:
    """The prefix under which the file stores the model's tensors: the candidate that
    makes the most wanted names resolve."""
    names = set(names)
    best, best_hits = prefixes[0], -1
    for p in prefixes:
        hits = sum(1 for w in wanted if p + w in names)
        if hits > best_hits:
            best, best_hits = p, hits
    return best


def _host_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float16, torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype in (torch.int64, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise WeightFileError(f"unsupported tensor dtype {t.dtype}")


def load_weights(model_dir: str, requests: Dict[str, TensorRequest],
                 prefixes: Sequence[str] = ("",),
                 ignored: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Open `model_dir/model.safetensors`, check it against `requests` and return the
    requested tensors by their un-prefixed names (host tensors, views of the mapping)."""
    path = os.path.join(model_dir, WEIGHT_FILE)
    if not os.path.isfile(path) and os.path.isfile(os.path.join(model_dir, WEIGHT_FILE + ".index.json")):
        raise WeightFileError(f"{model_dir}: sharded weight files (model.safetensors.index.json) are not supported")
    f = SafetensorsFile(path)
    prefix = _detect_prefix(f.names(), requests.keys(), list(prefixes) or [""])
    ignore_res = [re.compile(p) for p in ignored]

    missing, wrong_shape, wrong_kind = [], [], []
    for name, req in requests.items():
        full = prefix + name
        if full not in f:
            missing.append(full)
            continue
        got = f.shape(full)
        if tuple(got) != tuple(req.shape):
            wrong_shape.append((full, tuple(got), tuple(req.shape)))
        is_float = f.dtype(full).is_floating_point
        if is_float == req.integer:
            wrong_kind.append((full, str(f.dtype(full)).replace("torch.", "")))
    unexpected = []
    for full in f.names():
        bare = full[len(prefix):] if prefix and full.startswith(prefix) else full
        if bare in requests and (full == prefix + bare):
            continue
        if any(r.search(bare) for r in ignore_res) or any(r.search(full) for r in ignore_res):
            continue
        unexpected.append(full)
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightBindingError(path, sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(wrong_kind))

    out: Dict[str, torch.Tensor] = {}
    for name in requests:
        out[name] = _host_dtype(f.tensor(prefix + name))
    return out


def to_device(t: torch.Tensor, req: Optional[TensorRequest], device, compute_dtype: torch.dtype) -> torch.Tensor:
    """Move a loaded tensor to the device in the dtype the engine computes in."""
    if not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32).contiguous()
    if req is not None and req.keep_32bit and t.dtype == torch.float32:
        return t.to(device=device).contiguous()
    return t.to(device=device, dtype=compute_dtype).contiguous()
