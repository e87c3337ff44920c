from .params import SamplingParams

__all__ = ["SamplingParams", "Sampler"]


def __getattr__(name):
    if name == "Sampler":          # needs the CUDA library; loaded on first use
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
