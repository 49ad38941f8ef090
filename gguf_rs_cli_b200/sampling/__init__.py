from .params import SamplingParams, stream_key

__all__ = ["SamplingParams", "stream_key", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
