from .sampler import Sampler, SamplingParams, gumbel_noise, request_key

__all__ = ["Sampler", "SamplingParams", "gumbel_noise", "request_key"]
