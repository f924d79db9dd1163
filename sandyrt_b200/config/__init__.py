from .base import ConfigError, ModelConfig, load_config, save_config  # noqa: F401
from .gpt2 import GPT2Config  # noqa: F401
