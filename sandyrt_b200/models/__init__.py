"""Architectures shipped with the engine.  Importing this package registers them.
(The Model class lives in `models.model`; it is not imported here so that the parts,
which the model is built from, can import the spec types without a cycle.)"""
from . import gpt2  # noqa: F401
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec  # noqa: F401
