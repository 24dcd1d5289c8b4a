from .params import SamplingParams
from .sampler import Sampler, SampleRow

__all__ = ["SamplingParams", "Sampler", "SampleRow"]
