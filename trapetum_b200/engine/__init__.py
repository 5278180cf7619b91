from .engine import Engine, decode_splits
from .model import Model, load_model, parse_dtype, tensor_specs_for_config
from .step import StepContext, StepError

__all__ = ["Engine", "Model", "StepContext", "StepError", "decode_splits", "load_model", "parse_dtype",
           "tensor_specs_for_config"]
