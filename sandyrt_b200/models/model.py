"""Model: the parts of a ModelSpec built, bound to weights, and run over a step's tokens.

Building is three stages, each usable on its own:
  build_model(spec)            part objects from the spec (no weights, no device)
  model.tensor_requests()      every tensor the model wants, by name in the weight file
  model.bind(tensors, ...)     hand the loaded tensors to the parts and move them to the device
`load_model(dir, ...)` does all three from a model folder, choosing the architecture by
the folder's config.json.

`forward` runs the layer calls of the spec's schedule in order over the residual stream and
returns float32 logits at the wanted rows only (the reference computes every row,
src/models/gpt2_small.sandy.go:56-57; here the final norm and the head see just the rows
that were asked for).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ModelConfig, load_config
from ..parts.base import Block, LayerCallCtx, StepContext
from ..registry import get_architecture, get_part
from ..weights.loader import TensorRequest, load_weights
from .spec import LayerSpec, ModelSpec, PartSpec


def _build_block(layer: LayerSpec, width: int) -> Block:
    mixer = get_part("mixer", layer.mixer.kind)(layer.mixer)
    ff = get_part("feed_forward", layer.feed_forward.kind)(layer.feed_forward)
    norms = {name: get_part("norm", ps.kind)(ps) for name, ps in layer.norms.items()}
    block_cls = get_part("block", layer.block)
    missing = [n for n in getattr(block_cls, "norm_names", ()) if n not in norms]
    if missing:
        raise ValueError(f"block '{layer.block}' needs norms {missing}")
    return block_cls(mixer, ff, norms, width)


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = get_part("embedding", spec.embedding.kind)(spec.embedding)
        self.position = get_part("position", spec.position.kind)(spec.position)
        self.blocks: List[Block] = [_build_block(l, spec.width) for l in spec.layers]
        self.final_norm = get_part("norm", spec.final_norm.kind)(spec.final_norm)
        self.head = get_part("head", spec.head.kind)(spec.head)
        self.schedule = list(spec.schedule)
        for call in self.schedule:
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"run order names layer {call.layer}, the model has {len(self.blocks)}")
        self.device = None
        self.compute_dtype: Optional[torch.dtype] = None

    # ---- parts with their specs, for requests and binding -----------------------------
    def _parts(self):
        yield self.embedding, self.spec.embedding
        yield self.position, self.spec.position
        for block, layer in zip(self.blocks, self.spec.layers):
            yield block.mixer, layer.mixer
            yield block.feed_forward, layer.feed_forward
            for name, norm in block.norms.items():
                yield norm, layer.norms[name]
        yield self.final_norm, self.spec.final_norm
        yield self.head, self.spec.head

    def tensor_requests(self) -> Dict[str, TensorRequest]:
        """Name in the weight file -> expected shape, for every tensor the model reads."""
        out: Dict[str, TensorRequest] = {}
        for part, pspec in self._parts():
            for local, req in part.requests().items():
                if local not in pspec.tensors:
                    raise ValueError(f"{pspec.kind}: the model description names no tensor for '{local}'")
                name = pspec.tensors[local]
                if name in out and out[name].shape != req.shape:
                    raise ValueError(f"tensor '{name}' is requested with two shapes")
                out[name] = req
        return out

    def bind(self, tensors: Dict[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.device, self.compute_dtype = torch.device(device), dtype
        for part, pspec in self._parts():
            local = {l: tensors[pspec.tensors[l]] for l in part.requests()}
            if part is self.head:
                # a head that shares the token table says so with `tied`; it gets the bound table
                tied = getattr(self.head, "tied", False)
                part.bind(local, device, dtype, tied_weight=self.embedding.table() if tied else None)
            else:
                part.bind(local, device, dtype)

    # ---- cache needs ----------------------------------------------------------------------
    def cache_specs(self):
        """One cache spec per cache entry of the run order (None where a mixer keeps nothing)."""
        specs = [None] * self.spec.n_caches()
        for call in self.schedule:
            s = self.blocks[call.layer].mixer.cache_spec()
            if specs[call.cache] is not None and s != specs[call.cache]:
                raise ValueError(f"cache entry {call.cache} is used by layers with different needs")
            specs[call.cache] = s
        return specs

    @property
    def graph_safe(self) -> bool:
        """Whether every part may be recorded in a CUDA graph (see Part.graph_safe)."""
        return all(getattr(part, "graph_safe", True) for part, _ in self._parts())

    @property
    def max_positions(self) -> Optional[int]:
        return self.position.max_positions

    def weight_bytes(self) -> int:
        """Bytes of weights a decode step reads once: every layer call's parts and the head (each
        part reports its own; a part that reports nothing counts as 0)."""
        total = self.head.weight_bytes() + self.final_norm.weight_bytes()
        for call in self.schedule:
            b = self.blocks[call.layer]
            total += b.mixer.weight_bytes() + b.feed_forward.weight_bytes()
            total += sum(n.weight_bytes() for n in b.norms.values())
        return total

    # ---- the forward pass over one step's tokens ---------------------------------------
    def forward(self, ctx: StepContext, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        ws = ctx.workspace
        ctx.position = self.position
        x = ws.get("stream", ctx.n_tokens, self.spec.width, torch.float32)
        self.embedding.forward(ctx, x, status)
        for call in self.schedule:
            self.blocks[call.layer].forward(ctx, x, LayerCallCtx(call.cache, call.write_cache))
        n_rows = ctx.logit_rows.numel()
        logits = ws.get("logits", n_rows, self.spec.vocab_size, torch.float32)
        if n_rows:
            y = ws.get("final_normed", n_rows, self.spec.width, ctx.compute_dtype)
            self.final_norm.forward(ctx, x, y, rows=ctx.logit_rows)
            self.head.forward(ctx, y, logits)
        return logits


def build_model(spec: ModelSpec) -> Model:
    return Model(spec)


def describe(config: ModelConfig) -> ModelSpec:
    return get_architecture(config.architecture).describe(config)


def load_model(model_dir: str, device="cuda:0", dtype: torch.dtype = torch.bfloat16) -> Model:
    config = load_config(model_dir)
    spec = describe(config)
    model = build_model(spec)
    tensors = load_weights(model_dir, model.tensor_requests(), spec.name_prefixes, spec.ignored_tensors)
    model.bind(tensors, device, dtype)
    model.config = config
    return model
