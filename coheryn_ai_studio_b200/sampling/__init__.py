from .sampler import DeviceSampler, RequestSampler, SamplingParams, SplitMix64

__all__ = ["DeviceSampler", "RequestSampler", "SamplingParams", "SplitMix64"]
