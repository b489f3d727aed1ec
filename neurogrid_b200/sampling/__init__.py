from .sampler import DEFAULT_SEED, Sampler, SamplingParams, uniform_for
