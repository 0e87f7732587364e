from .config import GenerationConfig, SamplingParams
from .sampler import Sampler
