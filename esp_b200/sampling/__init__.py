from .sampler import SamplingParams, as_signed64, entropy_seed, skip_draws, splitmix64_next

__all__ = ["SamplingParams", "as_signed64", "entropy_seed", "skip_draws", "splitmix64_next"]
