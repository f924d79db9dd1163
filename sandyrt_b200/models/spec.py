"""ModelSpec: an architecture described as data.

An architecture's `describe(config)` returns one ModelSpec.  It lists, for every layer, which
mixer, feed-forward and norms the layer is made of (a part kind plus its sizes and constants,
chosen layer by layer), how the block arranges them, the names of the tensors in the weight file,
and the order in which layers run.  The engine builds the model from this description alone; no
part is told which model it is in.

The host library holds the same structure (core/spec.h) and reads and writes it as JSON; these
dataclasses are its Python form: what `describe` of a built-in architecture returns, and what an
architecture defined in Python hands over.

The reference writes the same information as a program in its own language
(src/models/gpt2_small.sandy.go:1-59: functions for attention, MLP and block, a loop over
`range(12)`, weight names through nested `weight_scope`s).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional, Sequence, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its sizes/constants, and where its tensors live.

    `tensors` maps the part's own tensor names ("qkv.weight") to names in the weight file
    ("h.3.attn.c_attn.weight")."""
    kind: str
    params: Dict[str, Any] = dataclasses.field(default_factory=dict)
    tensors: Dict[str, str] = dataclasses.field(default_factory=dict)

    def to_json(self) -> Dict[str, Any]:
        return {"kind": self.kind, "params": dict(self.params), "tensors": dict(self.tensors)}

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "PartSpec":
        return cls(j["kind"], dict(j.get("params") or {}), dict(j.get("tensors") or {}))


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and their norms."""
    block: str                       # registered block kind, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]       # the block kind names the norms it wants


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes ModelSpec.layers (a layer may be named by several calls: shared weights).
    `cache` names the cache entry the mixer works on.  With `write_cache` false the call appends
    nothing and only reads what an earlier call of this step wrote there (a layer that reads
    another layer's keys and values)."""
    layer: int
    cache: int
    write_cache: bool = True


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab_size: int
    max_positions: Optional[int]     # None when the position encoding sets no limit
    embedding: PartSpec              # token table ("weight": name)
    position: PartSpec               # position encoding
    layers: Sequence[LayerSpec]
    schedule: Sequence[LayerCall]
    final_norm: PartSpec
    head: PartSpec                   # params: tied (bool); tensors: "weight"
    # All names in `tensors` are written without these prefixes; a file may carry one of them on
    # every name (HF stores GPT-2 both as "transformer.h.0..." and "h.0...").
    name_prefixes: Tuple[str, ...] = ("",)
    # Regular expressions for tensors that a file may hold and the model does not read (buffers
    # such as a stored causal mask).
    ignored_tensors: Tuple[str, ...] = ()
    eos_token_id: Optional[int] = None

    def n_caches(self) -> int:
        return 1 + max((c.cache for c in self.schedule), default=-1)

    def to_json(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture, "width": self.width, "vocab_size": self.vocab_size,
            "max_positions": self.max_positions, "embedding": self.embedding.to_json(),
            "position": self.position.to_json(),
            "layers": [{"block": l.block, "mixer": l.mixer.to_json(), "feed_forward": l.feed_forward.to_json(),
                        "norms": {k: v.to_json() for k, v in l.norms.items()}} for l in self.layers],
            "schedule": [{"layer": c.layer, "cache": c.cache, "write_cache": c.write_cache} for c in self.schedule],
            "final_norm": self.final_norm.to_json(), "head": self.head.to_json(),
            "name_prefixes": list(self.name_prefixes), "ignored_tensors": list(self.ignored_tensors),
            "eos_token_id": self.eos_token_id,
        }

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "ModelSpec":
        return cls(
            architecture=j["architecture"], width=j["width"], vocab_size=j["vocab_size"],
            max_positions=j.get("max_positions"), embedding=PartSpec.from_json(j["embedding"]),
            position=PartSpec.from_json(j["position"]),
            layers=[LayerSpec(l["block"], PartSpec.from_json(l["mixer"]), PartSpec.from_json(l["feed_forward"]),
                              {k: PartSpec.from_json(v) for k, v in l["norms"].items()}) for l in j["layers"]],
            schedule=[LayerCall(c["layer"], c["cache"], c.get("write_cache", True)) for c in j["schedule"]],
            final_norm=PartSpec.from_json(j["final_norm"]), head=PartSpec.from_json(j["head"]),
            name_prefixes=tuple(j.get("name_prefixes") or ("",)), ignored_tensors=tuple(j.get("ignored_tensors") or ()),
            eos_token_id=j.get("eos_token_id"))
