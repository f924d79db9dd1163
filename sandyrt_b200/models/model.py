"""Model: a handle on a model built by the host library, and how one is made.

Building is three stages (core/model.cpp), each usable on its own:
  build_model(spec or config)   part objects from the description (no weights, no device)
  model.tensor_requests()       every tensor the model wants, by name in the weight file
  load_model(dir, ...)          all of it from a model folder, the architecture chosen by the
                                folder's config.json, weights bound and moved to the device

The forward pass runs the layer calls of the description's run order over the residual stream and
returns float32 logits at the wanted rows only (the reference computes every row,
src/models/gpt2_small.sandy.go:56-57; here the final norm and the head see just the rows that were
asked for).  It runs inside the library, under Engine.step.
"""
from __future__ import annotations

from typing import Dict, Optional, Union

import torch

from .. import core
from ..config.base import ModelConfig, config_from_normalised, load_config
from ..weights.loader import TensorRequest, requests_from_json
from .spec import ModelSpec

_DTYPE_NAMES = {torch.bfloat16: "bfloat16", torch.float32: "float32"}


class Model:
    def __init__(self, handle: core.Handle, config: Optional[ModelConfig] = None):
        self._h = handle
        self._info_method = "info"
        self.config = config
        self.spec = ModelSpec.from_json(handle.call("spec"))

    def tensor_requests(self) -> Dict[str, TensorRequest]:
        """Name in the weight file -> expected shape, for every tensor the model reads."""
        return requests_from_json(self._h.call("tensor_requests"))

    def _info(self):
        return self._h.call(self._info_method)

    def _handle_for_engine(self) -> int:
        """The library's model object, to hand to an engine; a model that an LLM has taken over is
        not one any more."""
        if self._h.kind != "model":
            raise ValueError("this model already belongs to an LLM: build or load another one for a second engine")
        return self._h.handle

    def _moved_into(self, owner: core.Handle) -> None:
        """An engine of the library has taken the model over: ask it from now on."""
        self._h = core.Handle(owner.kind, owner.handle, owned=False, keep=owner)
        self._info_method = "model_info"

    @property
    def graph_safe(self) -> bool:
        """Whether every part may be recorded in a CUDA graph."""
        return self._info()["graph_safe"]

    @property
    def max_positions(self) -> Optional[int]:
        return self._info()["max_positions"]

    @property
    def compute_dtype(self) -> torch.dtype:
        return getattr(torch, self._info()["dtype"])

    def weight_bytes(self) -> int:
        """Bytes of weights a decode step reads once: every layer call's parts and the head."""
        return self._info()["weight_bytes"]

    def bind_random(self, seed: int, dtype: torch.dtype, device: int = 0) -> None:
        """Bind seeded random weights (the random-weights mode without a folder in between)."""
        self._h.call("bind_random", seed=int(seed), dtype=_DTYPE_NAMES[dtype], device=device)


def describe(config: ModelConfig) -> ModelSpec:
    """The model description of a configuration: its architecture's `describe`."""
    return ModelSpec.from_json(core.call("global", None, "describe", config=config.to_dict()))


def build_model(what: Union[ModelSpec, ModelConfig]) -> Model:
    """The parts of a description (or of a configuration's description), without weights."""
    if isinstance(what, ModelSpec):
        return Model(core.Handle("model", core.call("global", None, "build_model_from_spec", spec=what.to_json())["handle"]))
    return Model(core.Handle("model", core.call("global", None, "build_model", config=what.to_dict())["handle"]), what)


def _device_index(device) -> int:
    d = torch.device(device)
    if d.type != "cuda":
        raise RuntimeError("sandyrt_b200 needs a CUDA device; there is no CPU path")
    return d.index or 0


def load_model(model_dir: str, device="cuda:0", dtype: torch.dtype = torch.bfloat16) -> Model:
    h = core.Handle("model", core.call("global", None, "load_model", model_dir=model_dir, dtype=_DTYPE_NAMES[dtype],
                                       device=_device_index(device))["handle"])
    cfg = h.call("config")
    return Model(h, config_from_normalised(cfg) if cfg else None)
