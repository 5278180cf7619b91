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
import os as _os

from .engine import Model
from .engine import Engine as _PythonEngine
from .engine import load_model as _python_load_model
from .engine import random_model as _python_random_model
from .parts import register_part
from .weights import WeightError, write_random_model

__version__ = "0.2.0"

HOSTS = ("python", "native")


def _host(host, config) -> str:
    """Which host runs a model.  "native": the C++ library (``trapetum_b200.native``), for models whose parts all
    have native classes; it refuses others.  "python": this package's own loop, which also runs parts written in
    Python.  "auto" (the default; or $TRAPETUM_HOST): native where the model allows it, else python."""
    host = host or _os.environ.get("TRAPETUM_HOST") or "auto"
    if host == "auto":
        from . import native
        return "native" if native.is_native(load_config(config)[1]) else "python"
    if host not in HOSTS:
        raise ValueError(f"host must be one of {HOSTS + ('auto',)}, got {host!r}")
    return host


def load_model(folder, dtype="bfloat16", device="cuda:0", fp16="widen", host=None):
    """Read config.json, pick the model by its architecture name, load and bind the weights."""
    if _host(host, folder) == "native":
        from . import native
        return native.load_model(folder, dtype, device, fp16)
    return _python_load_model(folder, dtype, device, fp16)


def random_model(config, seed=0, std=0.02, norm_std=0.1, dtype="bfloat16", device="cuda:0", host=None):
    """A model of ``config`` with random weights made on the device (the values that ``write_random_model`` stores)."""
    if _host(host, config) == "native":
        from . import native
        return native.random_model(config, seed, std, norm_std, dtype, device)
    return _python_random_model(config, seed, std, norm_std, dtype, device)


def _is_native(x) -> bool:
    import sys
    nat = sys.modules.get(__name__ + ".native")
    return nat is not None and isinstance(x, (nat.Model, nat.Engine))


def Engine(model, max_tokens, max_slots=None, use_graphs=True):
    """The engine of a model: its cache and the step function, on the host that holds the model."""
    if _is_native(model):
        from . import native
        return native.Engine(model, max_tokens, max_slots, use_graphs)
    return _PythonEngine(model, max_tokens, max_slots, use_graphs)


def generate(model_or_engine, *args, **kwargs):
    if _is_native(model_or_engine):
        from . import native
        return native.generate(model_or_engine, *args, **kwargs)
    from .engine.generate import generate as _g
    return _g(model_or_engine, *args, **kwargs)


__all__ = ["ConfigError", "Engine", "Model", "WeightError", "generate", "load_config", "load_model",
           "random_model", "register_architecture", "register_part", "write_random_model"]
