"""The host side of the sampler against the plain implementation, and the rule of one
uniform per sampled token."""

import numpy as np
import pytest

from sllm_b200.sampling import SamplingParams, apply_repetition_penalty, sample_host
from tests.plain import qwen2_plain as plain


def test_host_sampler_matches_plain():
    rng = np.random.default_rng(0)
    for trial in range(50):
        logits = rng.standard_normal(97) * 3
        for kw in (dict(temperature=0.7), dict(temperature=1.0, top_k=5), dict(temperature=1.3, top_p=0.8),
                   dict(temperature=0.9, top_k=20, top_p=0.5), dict(temperature=0.0)):
            a, b = np.random.default_rng(trial), np.random.default_rng(trial)
            got = sample_host(logits, SamplingParams(**kw), a)
            want = plain.sample(logits, kw["temperature"], kw.get("top_k"), kw.get("top_p"),
                                u=b.random() if kw["temperature"] > 0 else None)
            assert got == want
            if kw["temperature"] > 0:
                assert a.random() == b.random()                # exactly one uniform was drawn


def test_penalty_and_params():
    np.testing.assert_allclose(apply_repetition_penalty(np.array([2.0, -2.0, 1.0]), [0, 1, 99, -3], 2.0), [1, -4, 1])
    x = np.array([1.0, 2.0])
    assert apply_repetition_penalty(x, [0], 1.0) is not x
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
