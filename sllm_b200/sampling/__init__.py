from .params import SamplingParams
from .sampler import Sampler, apply_repetition_penalty, sample_host

__all__ = ["SamplingParams", "Sampler", "apply_repetition_penalty", "sample_host"]
