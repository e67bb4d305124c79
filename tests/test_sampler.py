"""The host side of the sampler: parameters, and the inputs the sampling kernel is given (one
uniform per sampled token, each seen id once)."""

import numpy as np
import pytest

from sllm_b200.sampling import SamplingParams


def test_penalty_and_params():
    with pytest.raises(ValueError):
        SamplingParams(top_k=0)
    with pytest.raises(ValueError):
        SamplingParams(max_new=0)
    assert not SamplingParams(temperature=0.8, top_p=0.9, top_k=3).penalised
    assert SamplingParams(repetition_penalty=1.1).penalised and not SamplingParams(repetition_penalty=1.0).penalised


def test_kernel_inputs_of_the_sampler():
    from sllm_b200.sampling.sampler import Sampler
    rows = [(SamplingParams(temperature=0.0, top_k=4), np.random.default_rng(0), None),
            (SamplingParams(temperature=0.7, top_k=4, top_p=0.5), np.random.default_rng(1), None),
            (SamplingParams(temperature=1.0, repetition_penalty=1.5), np.random.default_rng(2), [3, 9, 3, 1])]
    temps, unis, top_k, top_p = Sampler.host_inputs(rows)
    assert temps.tolist() == pytest.approx([0.0, 0.7, 1.0]) and top_k.tolist() == [0, 4, 0]
    assert top_p.tolist() == [-1.0, 0.5, -1.0]
    assert unis[0] == 0.0 and unis[1] == np.random.default_rng(1).random()       # a greedy row draws nothing
    r, t, q = Sampler.penalty_pairs(rows)
    assert r.tolist() == [2, 2, 2] and t.tolist() == [1, 3, 9] and q.tolist() == [1.5] * 3   # each id once
    assert Sampler.penalty_pairs(rows[:2]) is None
    assert Sampler.penalties([p for p, _, _ in rows]).tolist() == [1.0, 1.0, 1.5]
    assert Sampler.penalties([p for p, _, _ in rows[:2]]) is None
