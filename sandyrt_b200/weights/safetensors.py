"""Reader and writer for the safetensors container.

Format, as the reference reads it (src/weight/SafeTensorWeights.cpp:44-95 and its Python
twin scripts/run_gpt2.py:39-83): an unsigned 64-bit little-endian header length, a JSON
header `{name: {dtype, shape, data_offsets:[begin,end]}}` (the `__metadata__` entry is
skipped), then the payload; offsets are relative to the end of the header.  Dtypes
accepted are those of the reference's parse_dtype (:14-23): F32, F16, BF16, I32, I64, U8,
BOOL.  Where the reference aborts on a bad file, every fault here is a WeightFileError
that says what is wrong with which file.

The file is memory-mapped; a tensor is a zero-copy view until it is cast or moved.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
# A header larger than this is taken for a corrupt length field.
_MAX_HEADER_BYTES = 100 * 1024 * 1024


class WeightFileError(Exception):
    """The weight file is missing, truncated or not a well-formed safetensors file."""


class SafetensorsFile:
    """A memory-mapped safetensors file: `names()`, `shape(name)`, `tensor(name)`."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.isfile(path):
            raise WeightFileError(f"weight file not found: {path}")
        size = os.path.getsize(path)
        if size < 8:
            raise WeightFileError(f"{path}: {size} bytes is too short for a safetensors file")
        self._file = open(path, "rb")
        try:
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except (ValueError, OSError) as e:
            self._file.close()
            raise WeightFileError(f"{path}: cannot map file ({e})") from e
        (header_len,) = struct.unpack_from("<Q", self._map, 0)
        if header_len > _MAX_HEADER_BYTES or 8 + header_len > size:
            raise WeightFileError(
                f"{path}: header length {header_len} exceeds the file size {size} (truncated or corrupt)")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise WeightFileError(f"{path}: header must be a JSON object")
        self._data_start = 8 + header_len
        payload = size - self._data_start
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        spans = []
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (begin, end) = meta["dtype"], meta["shape"], meta["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise WeightFileError(f"{path}: malformed header entry for '{name}' ({e})") from e
            if dtype_name not in _DTYPES:
                raise WeightFileError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            numel = 1
            for d in shape:
                if not isinstance(d, int) or d < 0:
                    raise WeightFileError(f"{path}: tensor '{name}' has a bad shape {shape}")
                numel *= d
            if not (0 <= begin <= end <= payload):
                raise WeightFileError(
                    f"{path}: tensor '{name}' spans bytes [{begin},{end}) outside the payload of {payload} bytes")
            if end - begin != numel * width:
                raise WeightFileError(
                    f"{path}: tensor '{name}' has {end - begin} bytes, shape {shape} of {dtype_name} needs {numel * width}")
            self._entries[name] = (dtype, tuple(shape), begin, end)
            if end > begin:
                spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise WeightFileError(f"{path}: tensors '{n0}' and '{n1}' overlap in the payload")

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A view of the mapped bytes (read-only memory: clone or cast before writing)."""
        dtype, shape, begin, end = self._entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the mapped buffer is read-only
            flat = torch.frombuffer(self._map, dtype=dtype, count=(end - begin) // _DTYPES[_NAMES[dtype]][1],
                                    offset=self._data_start + begin)
        return flat.view(shape)

    def close(self) -> None:
        # Views handed out keep the mapping alive through the buffer protocol; closing is
        # only attempted, never forced.
        try:
            self._map.close()
        except BufferError:
            pass
        self._file.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write `tensors` (host tensors) as one safetensors file, names sorted, atomically."""
    header = {}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)  # keep the payload 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
