from .params import SamplingParams
from .sampler import Sampler, SampleTicket, uniform_from

__all__ = ["SamplingParams", "Sampler", "SampleTicket", "uniform_from"]
