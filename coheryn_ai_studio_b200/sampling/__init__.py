from .sampler import DeviceSampler, HostSampler, RequestSampler, SamplingParams, SplitMix64

__all__ = ["DeviceSampler", "HostSampler", "RequestSampler", "SamplingParams", "SplitMix64"]
