from .sampler import DeviceSampler, SamplingParams, stream_seed

__all__ = ["DeviceSampler", "SamplingParams", "stream_seed"]
