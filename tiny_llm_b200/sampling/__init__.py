from .params import SamplingParams
from .sampler import Sampler, uniform_from

__all__ = ["SamplingParams", "Sampler", "uniform_from"]
