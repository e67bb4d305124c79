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
    assert SamplingParams(temperature=0.8).on_device and not SamplingParams(top_p=0.9).on_device
    assert not SamplingParams(repetition_penalty=1.1).on_device and SamplingParams(repetition_penalty=1.0).on_device
