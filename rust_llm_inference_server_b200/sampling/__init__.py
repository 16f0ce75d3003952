from .params import SamplingParams
from .sampler import Sampler, filtered_draw, lowbias32, row_key, unit_uniform, unit_uniform_53
