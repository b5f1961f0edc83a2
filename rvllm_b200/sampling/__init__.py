from .params import GREEDY, SamplingParams
from .sampler import BatchSampler
