from .sampler import Sampler, request_seed

__all__ = ["Sampler", "request_seed"]
