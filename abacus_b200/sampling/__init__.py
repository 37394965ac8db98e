from .sampler import Sampler, stream_seed

__all__ = ["Sampler", "stream_seed"]
