"""Sampling: options, random streams and the device sampler."""
from .rng import XorShift128Plus, request_seed
from .sampler import GREEDY_BELOW, REPEAT_WINDOW, RequestSamplingState, Sampler, SamplingConfig

__all__ = ["XorShift128Plus", "request_seed", "GREEDY_BELOW", "REPEAT_WINDOW", "RequestSamplingState",
           "Sampler", "SamplingConfig"]
