from .sampler import RECENT_WINDOW, Sampler, SamplingOptions

__all__ = ["RECENT_WINDOW", "Sampler", "SamplingOptions"]
