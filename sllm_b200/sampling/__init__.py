from .params import SamplingParams
from .sampler import Sampler

__all__ = ["SamplingParams", "Sampler"]
