from .params import SamplingParams, GREEDY, RANDOM, TOP_K, TOP_P
from .sampler import Sampler, uniform_for
