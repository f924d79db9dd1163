"""Binding of the host library (core/*.cpp -> libsandy_core.so, its C interface in core/c_api.h).

Everything the engine does on the host (configuration, model descriptions, weights, the cache
manager, the step function, the scheduler, generation) lives in that library; the Python package is
its face: argument conversion, exceptions, and parts or architectures that a caller defines in
Python and registers through the library's callbacks.

`call(object, handle, method, **args)` is the structured control plane (JSON in, JSON out); the hot
paths have typed functions on `lib()`.
"""
from __future__ import annotations

import ctypes
import json
import os
import threading
from typing import Any, Optional

from . import errors
from .csrc import build

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()
_pending_exception: Optional[BaseException] = None      # raised by a Python callback while the library ran


class TensorView(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int), ("rows", ctypes.c_longlong),
                ("cols", ctypes.c_longlong), ("ld", ctypes.c_longlong)]


class StepView(ctypes.Structure):
    _fields_ = [("n_tokens", ctypes.c_int), ("n_seqs", ctypes.c_int), ("n_rows", ctypes.c_int),
                ("max_blocks", ctypes.c_int), ("max_q_len", ctypes.c_int), ("max_kv_len", ctypes.c_int),
                ("compute_dtype", ctypes.c_int), ("n_groups", ctypes.c_int),
                ("token_ids", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("token_seq", ctypes.c_void_p),
                ("seq_slots", ctypes.c_void_p), ("q_start", ctypes.c_void_p), ("kv_before", ctypes.c_void_p),
                ("logit_rows", ctypes.c_void_p), ("block_tables", ctypes.POINTER(ctypes.c_void_p)),
                ("host_q_lens", ctypes.POINTER(ctypes.c_int)), ("host_kv_before", ctypes.POINTER(ctypes.c_int)),
                ("host_slots", ctypes.POINTER(ctypes.c_int)), ("stream", ctypes.c_void_p), ("context", ctypes.c_void_p)]


JSON_FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p)
TOKEN_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int)
PROVIDER_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int)
CREATE_FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p)
DESTROY_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p)
TEXT_FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p)
BIND_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p,
                           ctypes.c_char_p, ctypes.POINTER(ctypes.c_longlong), ctypes.c_int, ctypes.c_int)
FORWARD_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(StepView),
                              ctypes.POINTER(TensorView), ctypes.POINTER(TensorView), ctypes.c_int, ctypes.c_int,
                              ctypes.POINTER(ctypes.c_int), ctypes.c_int)


class ForeignPart(ctypes.Structure):
    _fields_ = [("create", CREATE_FN), ("destroy", DESTROY_FN), ("requests", TEXT_FN), ("info", TEXT_FN),
                ("bind", BIND_FN), ("forward", FORWARD_FN)]


@PROVIDER_FN
def _provide_kernel(name, dir_buf, capacity):
    """The library asks for a kernel library that is not loaded yet: build it if it is missing or stale."""
    try:
        n = name.decode()
        if not build.is_current(n):
            build.compile_library(n)
        path = os.path.dirname(build.library_path(n)).encode() + b"\0"
        if len(path) > capacity:
            return 1
        ctypes.memmove(dir_buf, path, len(path))
        return 0
    except BaseException as e:      # the build error is shown where the library's own error is raised
        remember_exception(e)
        return 1


def remember_exception(e: BaseException) -> None:
    global _pending_exception
    _pending_exception = e


def lib() -> ctypes.CDLL:
    """The loaded host library (built at first use)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        l = build.load_core()
        for name in ("sandy_last_error_kind", "sandy_last_error_message", "sandy_last_error_details", "sandy_call",
                     "sandy_llm_generate"):
            getattr(l, name).restype = ctypes.c_char_p
        for name in ("sandy_llm_load", "sandy_llm_from_model", "sandy_llm_engine", "sandy_engine_stream"):
            getattr(l, name).restype = ctypes.c_void_p
        l.sandy_llm_add_request.restype = ctypes.c_longlong
        l.sandy_kernel_launches.restype = ctypes.c_longlong
        l.sandy_engine_elapsed_ms.restype = ctypes.c_float
        l.sandy_release.restype = None
        l.sandy_set_kernel_provider(_provide_kernel)
        _lib = l
    return _lib


def raise_last_error() -> None:
    """Raise the calling thread's last library error (or the Python exception a callback left)."""
    global _pending_exception
    l = lib()
    kind = l.sandy_last_error_kind().decode()
    message = l.sandy_last_error_message().decode("utf-8", "replace")
    details = l.sandy_last_error_details().decode("utf-8", "replace")
    pending, _pending_exception = _pending_exception, None
    if pending is not None:
        raise pending
    cls = errors.KINDS.get(kind, RuntimeError)
    if cls is errors.WeightBindingError:
        raise cls(message, details)
    raise cls(message)


def call(obj: str, handle: Optional[int], method: str, **args: Any) -> Any:
    """One call of the structured control plane; returns the decoded result."""
    text = lib().sandy_call(obj.encode(), ctypes.c_void_p(handle or 0), method.encode(), json.dumps(args).encode())
    if text is None:
        raise_last_error()
    return json.loads(text)


class Handle:
    """An object of the host library; given back when the Python object goes away."""

    def __init__(self, kind: str, handle: int, owned: bool = True, keep: Any = None):
        self.kind, self.handle, self.owned, self.keep = kind, handle, owned, keep

    def call(self, method: str, **args: Any) -> Any:
        return call(self.kind, self.handle, method, **args)

    def __del__(self):
        try:
            if self.owned and self.handle and _lib is not None:
                _lib.sandy_release(self.kind.encode(), ctypes.c_void_p(self.handle))
        except Exception:
            pass
        self.handle = 0


def launches() -> int:
    """Kernel launches issued by the host library so far."""
    return int(lib().sandy_kernel_launches())
