from .params import SamplingParams
from .sampler import Sampler, request_seed, splitmix64

__all__ = ["SamplingParams", "Sampler", "request_seed", "splitmix64"]
