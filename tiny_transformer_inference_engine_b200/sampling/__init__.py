from .params import SamplingParams
from .sampler import Sampler, STATE_WORDS

__all__ = ["SamplingParams", "Sampler", "STATE_WORDS"]
