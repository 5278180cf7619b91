from .engine import Engine, len_bucket
from .model import Model, load_model, parse_dtype, random_model, tensor_specs_for_config
from .step import StepContext, StepError

__all__ = ["Engine", "Model", "StepContext", "StepError", "len_bucket", "load_model", "parse_dtype", "random_model",
           "tensor_specs_for_config"]
