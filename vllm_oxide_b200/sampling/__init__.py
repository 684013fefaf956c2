from .params import SamplingParams
from .sampler import Sampler, row_key

__all__ = ["SamplingParams", "Sampler", "row_key"]
