from .params import SamplingParams
from .sampler import noise_uniform
