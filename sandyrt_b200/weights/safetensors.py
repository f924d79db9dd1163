"""The safetensors container, as torch tensors.

The reader and the writer are the host library's (core/safetensors.cpp: memory-mapped file, header
checks, every fault a WeightFileError that says what is wrong with which file); this module hands
its tensors to Python as torch views of the mapping and takes torch tensors to write.

Format, as the reference reads it (src/weight/SafeTensorWeights.cpp:44-95 and its Python twin
scripts/run_gpt2.py:39-83): an unsigned 64-bit little-endian header length, a JSON header
`{name: {dtype, shape, data_offsets:[begin,end]}}` (the `__metadata__` entry is skipped), then the
payload.  Dtypes: F32, F16, BF16, I32, I64, U8, BOOL (the reference's parse_dtype, :14-23).
"""
from __future__ import annotations

import ctypes
import warnings
from typing import Any, Dict, Iterable, Tuple

import torch

from .. import core
from ..errors import WeightFileError  # noqa: F401  (re-exported)

_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I32": torch.int32,
           "I64": torch.int64, "U8": torch.uint8, "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


def tensor_at(entry: Dict[str, Any], keep: Any) -> torch.Tensor:
    """A torch view of host memory the library holds (`keep` must outlive the view)."""
    dtype, shape, n = _DTYPES[entry["dtype"]], tuple(entry["shape"]), entry["bytes"]
    if n == 0:
        return torch.empty(shape, dtype=dtype)
    raw = (ctypes.c_char * n).from_address(entry["address"])
    raw._keep = keep                             # torch holds `raw`, `raw` holds the mapping: it lives as long as any view
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")          # torch warns that the mapped buffer is read-only
        return torch.frombuffer(raw, dtype=dtype, count=n // torch.empty((), dtype=dtype).element_size()).view(shape)


class SafetensorsFile:
    """A memory-mapped safetensors file: `names()`, `shape(name)`, `dtype(name)`, `tensor(name)`."""

    def __init__(self, path: str):
        self.path = path
        self._handle = core.Handle("weights", core.call("global", None, "open_weights", path=path)["handle"])
        self._entries: Dict[str, Dict[str, Any]] = self._handle.call("tensors")

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A view of the mapped bytes (read-only memory: clone or cast before writing)."""
        return tensor_at(self._entries[name], self._handle)

    def close(self) -> None:
        """Views handed out keep the mapping alive; nothing is forced."""


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write `tensors` (host tensors) as one safetensors file, names sorted, atomically."""
    held, table = [], {}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        held.append(t)
        table[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "address": t.data_ptr() if t.numel() else 0}
    core.call("global", None, "write_safetensors", path=path, tensors=table)
