from .params import DEFAULT_RANDOM_SEED, ResolvedParams, SamplingParams, ValidationError
from .sampler import Sampler
