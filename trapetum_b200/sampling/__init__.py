from .params import REPETITION_WINDOW, SamplingParams, draw_uniform
from .sampler import Sampler

__all__ = ["REPETITION_WINDOW", "SamplingParams", "Sampler", "draw_uniform"]
