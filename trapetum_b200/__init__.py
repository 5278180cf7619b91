"""trapetum_b200: a small generation library for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed
configuration and an architecture registry, weights by tensor name, layers put
together from parts, a paged cache with slots, one step function, a generation
loop, sampling, trace replay, and hand-written CUDA kernels underneath.

    import trapetum_b200 as tb
    model = tb.load_model("path/to/folder", dtype="bfloat16")
    out = tb.generate(model, prompts=[[2, 651, 6037]], max_tokens=24)
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, load_config, register_architecture
from .engine import Engine, Model, load_model, random_model
from .parts import register_part
from .weights import WeightError, write_random_model

__version__ = "0.1.0"


def generate(*args, **kwargs):
    from .engine.generate import generate as _g
    return _g(*args, **kwargs)


__all__ = ["ConfigError", "Engine", "Model", "WeightError", "generate", "load_config", "load_model",
           "random_model", "register_architecture", "register_part", "write_random_model"]
