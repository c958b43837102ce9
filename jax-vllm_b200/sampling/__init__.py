from .sampler import Sampler, mix64, uniform

__all__ = ["Sampler", "mix64", "uniform"]
