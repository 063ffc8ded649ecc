from .sampler import DEFAULT_SEED, Lcg, SamplingParams, ranked_sample, sample

__all__ = ["DEFAULT_SEED", "Lcg", "SamplingParams", "ranked_sample", "sample"]
