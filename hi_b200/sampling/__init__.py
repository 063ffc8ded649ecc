from .sampler import DEFAULT_SEED, Lcg, SamplingParams, ranked_sample, sample, sample_on_host

__all__ = ["DEFAULT_SEED", "Lcg", "SamplingParams", "ranked_sample", "sample", "sample_on_host"]
