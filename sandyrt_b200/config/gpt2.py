"""GPT2Config: the typed form of a GPT-2 config.json.

Keys and defaults follow the reference's artefact experiments/gpt2_small/config.json:1-30
(n_layer :16, n_embd :14, n_head :15, n_positions :17, vocab_size :30,
layer_norm_epsilon :11, activation_function :2, architectures :3-5, bos/eos :7,9).
Keys that file does not carry get the architecture's usual defaults:
n_inner (null -> 4 * n_embd), scale_attn_weights (true),
scale_attn_by_inverse_layer_idx (false), tie_word_embeddings (true).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional

from .base import ConfigError, ModelConfig, _require

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
        n_positions = _require(raw, "n_positions", int, default=None)
        if n_positions is None:
            # `n_ctx` is the legacy duplicate of n_positions (config.json:13).
            n_positions = _require(raw, "n_ctx", int)
        cfg = cls(
            n_layer=_require(raw, "n_layer", int),
            n_embd=_require(raw, "n_embd", int),
            n_head=_require(raw, "n_head", int),
            n_positions=n_positions,
            vocab_size=_require(raw, "vocab_size", int),
            n_inner=_require(raw, "n_inner", int, default=None),
            layer_norm_epsilon=_require(raw, "layer_norm_epsilon", float, default=1e-5),
            activation_function=_require(raw, "activation_function", str, default="gelu_new"),
            scale_attn_weights=_require(raw, "scale_attn_weights", bool, default=True),
            scale_attn_by_inverse_layer_idx=_require(
                raw, "scale_attn_by_inverse_layer_idx", bool, default=False),
            tie_word_embeddings=_require(raw, "tie_word_embeddings", bool, default=True),
            bos_token_id=_require(raw, "bos_token_id", int, default=None),
            eos_token_id=_require(raw, "eos_token_id", int, default=None),
        )
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "gpt2"
        return d

    def validate(self) -> None:
        for key in ("n_layer", "n_embd", "n_head", "n_positions", "vocab_size"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be > 0, got {getattr(self, key)}")
        if self.n_inner is not None and self.n_inner <= 0:
            raise ConfigError(f"config.json: 'n_inner' must be > 0, got {self.n_inner}")
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"config.json: n_embd ({self.n_embd}) is not divisible by n_head ({self.n_head})")
        if self.activation_function not in ACTIVATIONS:
            raise ConfigError(
                f"config.json: activation_function '{self.activation_function}' is not one of "
                f"{list(ACTIVATIONS)}")
        if not (self.layer_norm_epsilon > 0.0):
            raise ConfigError("config.json: layer_norm_epsilon must be > 0")
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None and not (0 <= v < self.vocab_size):
                raise ConfigError(f"config.json: {key}={v} is outside the vocabulary")
