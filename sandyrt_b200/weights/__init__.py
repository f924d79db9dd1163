from .loader import TensorRequest, WeightBindingError, load_weights  # noqa: F401
from .random_init import random_tensors, write_random_model  # noqa: F401
from .safetensors import SafetensorsFile, WeightFileError, write_safetensors  # noqa: F401
