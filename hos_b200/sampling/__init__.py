from .sampler import Sampler, SamplingParams, next_rand, stream_seed  # noqa: F401
