"""Model descriptions and the Model handle.  The architectures shipped with the engine (GPT-2) are
described by the host library (core/config.cpp, describe_gpt2)."""
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec  # noqa: F401
