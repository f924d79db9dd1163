"""GPT2Config: the typed form of a GPT-2 config.json.

Keys and defaults follow the reference's artefact experiments/gpt2_small/config.json:1-30
(n_layer :16, n_embd :14, n_head :15, n_positions :17, vocab_size :30, layer_norm_epsilon :11,
activation_function :2, architectures :3-5, bos/eos :7,9).  Keys that file does not carry get the
architecture's usual defaults: n_inner (null -> 4 * n_embd), scale_attn_weights (true),
scale_attn_by_inverse_layer_idx (false), tie_word_embeddings (true).

The reading of the keys and the checks on them are the host library's (core/config.cpp,
GPT2Config); this dataclass carries the result.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional

from .. import core
from .base import ModelConfig

ACTIVATIONS = ("gelu_new", "gelu")


@dataclasses.dataclass(frozen=True)
class GPT2Config(ModelConfig):
    architecture = "GPT2LMHeadModel"

    n_layer: int = 0
    n_embd: int = 0
    n_head: int = 0
    n_positions: int = 0
    vocab_size: int = 0
    n_inner: Optional[int] = None
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu_new"
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    tie_word_embeddings: bool = True
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    # ---- derived sizes -------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    # ---- json ----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GPT2Config":
        """Type checks and defaults only; `validate` checks the sizes against one another."""
        n = core.call("global", None, "parse_config", config=raw, architecture=cls.architecture, validate=False)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in n.items() if k in names})

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "gpt2"
        return d

    def validate(self) -> None:
        core.call("global", None, "parse_config", config=self.to_dict(), architecture=self.architecture, validate=True)
