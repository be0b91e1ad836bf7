from .sampler import Sampler, validate_sampling

__all__ = ["Sampler", "validate_sampling"]
