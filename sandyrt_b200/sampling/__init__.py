from .params import SamplingParams  # noqa: F401
from .sampler import fresh_seed, uniform_for  # noqa: F401
