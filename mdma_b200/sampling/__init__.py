from .params import SamplingParams, uniform

__all__ = ["SamplingParams", "uniform", "DeviceSampler"]


def __getattr__(name):
    if name == "DeviceSampler":
        from .sampler import DeviceSampler
        return DeviceSampler
    raise AttributeError(name)
