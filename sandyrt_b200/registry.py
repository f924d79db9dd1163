"""Registries: architecture name -> model description, and part kind -> part class.

The reference picks a model by an if/else chain over an `architecture` string
(src/server/Model.cpp:100-160, unknown -> "unknown model architecture: X").  Here both the
architectures and the parts they are built from are entries of open tables in the host library
(core/config.cpp, core/parts.cpp), so a new mixer, feed-forward, norm, position encoding or whole
architecture is added by registering it; no file of the framework changes.

What is registered here is defined in Python: the library receives callbacks and uses them exactly
as it uses its own C++ entries (which `architectures()` and `part_kinds()` list beside them).
"""
from __future__ import annotations

import ctypes
import dataclasses
import json
from typing import Any, Callable, Dict, List, Optional, Type

import torch

from . import core
from .config.base import ConfigError, ModelConfig


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    # describe(config) -> ModelSpec (see models/spec.py): the parts of every layer, the order in
    # which layers run, and the names of the tensors in the weight file.  None for architectures
    # of the library itself (models.model.describe asks the library).
    describe: Optional[Callable[[ModelConfig], "object"]]


_PY_ARCHITECTURES: Dict[str, Architecture] = {}
_PY_PARTS: Dict[str, Dict[str, type]] = {k: {} for k in ("mixer", "feed_forward", "norm", "position")}
_KEEP: List[Any] = []            # callbacks and strings the library holds pointers to


def _builtin_config_classes() -> Dict[str, Type[ModelConfig]]:
    from .config.gpt2 import GPT2Config

    return {GPT2Config.architecture: GPT2Config}


def _text(s: str) -> int:
    """A C string that stays alive (the library reads it after the callback returns)."""
    buf = ctypes.create_string_buffer(s.encode())
    _KEEP.append(buf)
    if len(_KEEP) > 4096:
        del _KEEP[:1024]
    return ctypes.addressof(buf)


def _fail(e: BaseException) -> None:
    core.remember_exception(e)
    core.lib().sandy_set_callback_error(type(e).__name__.encode(), str(e).encode())


# ---- architectures ----------------------------------------------------------------------------
def register_architecture(name: str, config_cls: Type[ModelConfig], describe) -> None:
    """Register an architecture defined in Python: its typed configuration class (from_dict,
    to_dict, validate) and `describe(config) -> ModelSpec`."""
    arch = Architecture(name, config_cls, describe)

    @core.JSON_FN
    def parse(_user, raw):
        try:
            cfg = config_cls.from_dict(json.loads(raw))
            cfg.validate()
            return _text(json.dumps(cfg.to_dict()))
        except BaseException as e:
            _fail(e)
            return None

    @core.JSON_FN
    def describe_cb(_user, normalised):
        try:
            cfg = config_cls.from_dict(json.loads(normalised))
            return _text(json.dumps(describe(cfg).to_json()))
        except BaseException as e:
            _fail(e)
            return None

    _KEEP.extend([parse, describe_cb])
    if core.lib().sandy_register_architecture(name.encode(), parse, describe_cb, None) != 0:
        core.raise_last_error()
    _PY_ARCHITECTURES[name] = arch


def get_architecture(name: str) -> Architecture:
    if name in _PY_ARCHITECTURES:
        return _PY_ARCHITECTURES[name]
    core.call("global", None, "get_architecture", name=name)          # unknown -> ConfigError listing the known ones
    cls = _builtin_config_classes().get(name)
    if cls is None:
        raise ConfigError(f"architecture {name!r} is known to the library but has no Python configuration class")
    return Architecture(name, cls, None)


def architectures() -> List[str]:
    return sorted(core.call("global", None, "architectures"))


# ---- parts -------------------------------------------------------------------------------------
_STORE = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I32": torch.int32, "I64": torch.int64,
          "U8": torch.uint8, "BOOL": torch.bool}
_COMPUTE = {0: torch.float32, 1: torch.bfloat16}


class _Instances:
    """The live instances of Python parts, by the integer the library knows them by."""

    def __init__(self):
        self.by_id: Dict[int, Any] = {}
        self.pending: Dict[int, Dict[str, torch.Tensor]] = {}
        self.next = 1


_instances = _Instances()


def register_part(family: str, kind: str, cls: type) -> None:
    """Register class `cls` (a subclass of parts.base.Mixer, FeedForward, Norm or PositionEncoding)
    as the implementation of part `kind` in `family`."""
    if family not in _PY_PARTS:
        raise KeyError(f"parts of family {family!r} cannot be defined in Python; one of {sorted(_PY_PARTS)} "
                       "(embeddings, heads and blocks are registered in C++)")
    from .models.spec import PartSpec
    from .parts import base

    @core.CREATE_FN
    def create(_user, spec_json):
        try:
            inst = cls(PartSpec.from_json(json.loads(spec_json)))
            i = _instances.next
            _instances.next += 1
            _instances.by_id[i] = inst
            return i
        except BaseException as e:
            _fail(e)
            return None

    @core.DESTROY_FN
    def destroy(_user, i):
        _instances.by_id.pop(i, None)
        _instances.pending.pop(i, None)

    @core.TEXT_FN
    def requests(_user, i):
        try:
            inst = _instances.by_id[i]
            out = {name: {"shape": list(r.shape), "init": r.init, "integer": r.integer, "keep_32bit": r.keep_32bit}
                   for name, r in inst.requests().items()}
            return _text(json.dumps(out))
        except BaseException as e:
            _fail(e)
            return None

    @core.TEXT_FN
    def info(_user, i):
        try:
            inst = _instances.by_id[i]
            out = {"graph_safe": bool(getattr(inst, "graph_safe", True)), "weight_bytes": int(inst.weight_bytes()),
                   "rotates": bool(getattr(inst, "rotates", False)), "max_positions": getattr(inst, "max_positions", None),
                   "cache": base.cache_spec_json(inst.cache_spec()) if hasattr(inst, "cache_spec") else None}
            return _text(json.dumps(out))
        except BaseException as e:
            _fail(e)
            return None

    @core.BIND_FN
    def bind(_user, i, name, host_data, store_dtype, shape, rank, compute_dtype):
        try:
            inst = _instances.by_id[i]
            dims = tuple(shape[k] for k in range(rank))
            dt = _STORE[store_dtype.decode()]
            n = 1
            for d in dims:
                n *= d
            if n:
                raw = (ctypes.c_char * (n * torch.empty((), dtype=dt).element_size())).from_address(host_data)
                t = torch.frombuffer(raw, dtype=dt, count=n).view(dims).clone()     # the library's memory: copy
            else:
                t = torch.empty(dims, dtype=dt)
            got = _instances.pending.setdefault(i, {})
            got[name.decode()] = t
            if len(got) == len(inst.requests()):           # the last of its tensors: hand them over
                inst.bind(_instances.pending.pop(i), "cuda", _COMPUTE[compute_dtype])
            return 0
        except BaseException as e:
            _fail(e)
            return 1

    @core.FORWARD_FN
    def forward(_user, i, step, a, b, cache, write_cache, rows, n_rows):
        try:
            inst = _instances.by_id[i]
            ctx = base.StepContext(step)
            with torch.cuda.stream(torch.cuda.ExternalStream(ctx.stream)):
                ta = base.wrap_view(a.contents) if a else None
                tb = base.wrap_view(b.contents) if b else None
                if family == "mixer":
                    inst.forward(ctx, ta, tb, base.LayerCallCtx(cache, bool(write_cache)))
                elif family == "feed_forward":
                    inst.forward(ctx, ta, tb)
                elif family == "norm":
                    r = None
                    if rows:
                        r = base.wrap_device(ctypes.cast(rows, ctypes.c_void_p).value, (n_rows,), 2)
                    inst.forward(ctx, ta, tb[:n_rows] if tb is not None else None, rows=r)
                else:
                    inst.rotate(ctx, ta, tb)
            return 0
        except BaseException as e:
            _fail(e)
            return 1

    vt = core.ForeignPart(create, destroy, requests, info, bind, forward)
    _KEEP.append(vt)
    if core.lib().sandy_register_part(family.encode(), kind.encode(), ctypes.byref(vt), None) != 0:
        core.raise_last_error()
    _PY_PARTS[family][kind] = cls


def get_part(family: str, kind: str) -> type:
    """The Python class registered for a kind.  Kinds of the library itself have no Python class:
    they are built inside the library from a model description (or, alone, by parts.harness)."""
    if kind in _PY_PARTS.get(family, {}):
        return _PY_PARTS[family][kind]
    core.call("global", None, "check_part_kind", family=family, kind=kind)      # unknown -> ConfigError
    raise ConfigError(f"{family} kind {kind!r} is implemented in the host library; it has no Python class")


def part_kinds(family: str) -> List[str]:
    return sorted(core.call("global", None, "part_kinds", family=family))
