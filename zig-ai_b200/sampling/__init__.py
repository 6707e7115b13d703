from .sampler import Sampler, SamplingParams, uniform
