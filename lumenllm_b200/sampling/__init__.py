from .sampler import DeviceSampler, SamplingConfig, fresh_seed, uniform

__all__ = ["DeviceSampler", "SamplingConfig", "fresh_seed", "uniform"]
