from .params import SamplingParams
from .sampler import Sampler, SampleRow, SamplerOutput

__all__ = ["SamplingParams", "Sampler", "SampleRow", "SamplerOutput"]
