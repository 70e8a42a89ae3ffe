from .sampler import Rng, SamplingParams, sample_host, argmax_first
