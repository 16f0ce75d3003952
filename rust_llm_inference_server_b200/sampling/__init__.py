from .params import SamplingParams
from .sampler import Sampler, lowbias32, row_key, unit_uniform
