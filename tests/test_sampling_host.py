"""The host half of sampling (CPU): generator, parameter checks, ranked sampler."""
import numpy as np
import pytest
import torch

import plain_llama4 as plain
from hi_b200.sampling import Lcg, SamplingParams, ranked_sample


def test_generator_matches_the_plain_one():
    a, b = Lcg(0x4849), plain.Lcg(0x4849)
    xs = [a.next_f32() for _ in range(50)]
    assert xs == [b.next_f32() for _ in range(50)] and all(0 <= x < 1 for x in xs) and len(set(xs)) == 50


def test_ranked_sampler_matches_the_plain_one():
    rng = np.random.default_rng(0)
    for trial in range(200):
        v = int(rng.integers(2, 300))
        row = (rng.standard_normal(v) * 3).astype(np.float32)
        if trial % 7 == 0:
            row[rng.integers(0, v)] = row.max()                 # a tie at the top
        temp = float(rng.uniform(0.3, 2.0))
        top_p = float(rng.choice([1.0, 0.95, 0.5, 0.1]))
        top_k = int(rng.choice([0, 1, 5, 50]))
        if top_p >= 1.0 and not (0 < top_k < v):
            top_k = 1 + trial % 3
        u = float(rng.uniform())
        assert ranked_sample(row, temp, top_p, top_k or None, u) == plain.sample(torch.from_numpy(row), temp, top_p, top_k, u)


def test_params():
    assert SamplingParams().greedy and not SamplingParams().ranked(100)
    assert SamplingParams(temperature=0.8).ranked(100) is False
    assert SamplingParams(temperature=0.8, top_p=0.9).ranked(100) and SamplingParams(temperature=0.8, top_k=5).ranked(100)
    assert not SamplingParams(temperature=0.8, top_k=100).ranked(100)
    for bad in (dict(max_tokens=0), dict(temperature=float("nan")), dict(top_p=-0.1), dict(top_k=0)):
        with pytest.raises(ValueError, match="invalid_request_parameter"):
            SamplingParams(**bad).validate()
