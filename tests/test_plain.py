"""The plain implementation against logits that the reference project's own model
code produced (tests/golden/make_golden.py), and its own internal consistency."""

import os

import numpy as np
import pytest

from tests.golden.make_golden import CASES, golden_ids, golden_weights
from tests.plain import qwen2_plain as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "qwen2_tiny_golden.npz")


def _cfg(c):
    c = dict(c)
    c.setdefault("partial_rotary_factor", 1.0)
    return c


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_matches_reference_golden(name):
    gold = np.load(GOLDEN)
    cfg, seed, std, lengths = CASES[name]
    w = golden_weights(cfg, seed, std)
    for n in lengths:
        ids = golden_ids(cfg, seed, n)
        got = plain.forward(ids, w, _cfg(cfg))
        np.testing.assert_allclose(got, gold[f"{name}_{n}_full"], rtol=1e-6, atol=1e-6)
        if n > 4:
            # the reference's cached path gives the same rows as a whole forward
            np.testing.assert_allclose(got[n - 4:], gold[f"{name}_{n}_cached"], rtol=1e-5, atol=1e-6)


def test_causality_of_plain():
    cfg, seed, std, _ = CASES["A"]
    w = golden_weights(cfg, seed, std)
    ids = golden_ids(cfg, seed, 20)
    full = plain.forward(ids, w, _cfg(cfg))
    part = plain.forward(ids[:11], w, _cfg(cfg))
    np.testing.assert_allclose(full[:11], part, rtol=1e-6, atol=1e-6)


def test_sampler_plain():
    rng = np.random.default_rng(0)
    logits = rng.standard_normal(50)
    assert plain.greedy(logits) == int(np.argmax(logits))
    assert plain.sample(logits, temperature=0.0) == plain.greedy(logits)
    # top_k=1 is greedy whatever the uniform
    assert plain.sample(logits, 1.0, top_k=1, u=0.99) == plain.greedy(logits)
    # inverse CDF: u=0 gives the first token with non-zero mass
    assert plain.sample(logits, 1.0, u=0.0) == 0
    p = plain.apply_repetition_penalty(np.array([2.0, -2.0, 1.0]), [0, 1, 7], 2.0)
    np.testing.assert_allclose(p, [1.0, -4.0, 1.0])
    with pytest.raises(ValueError):
        plain.sample(logits, 1.0, top_k=0, u=0.5)
