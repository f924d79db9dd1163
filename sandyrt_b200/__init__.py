"""sandyrt_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and architecture registry, weights bound by name, layers put together from
parts, a paged cache manager, one step function for mixed batches, a scheduler, samplers,
hand-written CUDA kernels, a true 32-bit path, and a trace-replay tool.
"""
__version__ = "0.1.0"


def __getattr__(name):
    # heavy imports on first use only
    if name in ("LLM", "SamplingParams", "GenerateResult"):
        from .engine import llm
        return getattr(llm, name)
    raise AttributeError(name)
