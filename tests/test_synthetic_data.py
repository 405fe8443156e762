"""The synthetic dataset must give independent streams per example (no shifted copies)."""
import math

import numpy as np

from levanter_b200.data.synthetic import SyntheticLmDataset


def _ngrams(a, n=16):
    return {tuple(a[i:i + n]) for i in range(len(a) - n + 1)}


def test_examples_share_no_16_gram():
    ds = SyntheticLmDataset(32000, 4096, seed=0)
    prev = _ngrams(ds.tokens_at(0).numpy())
    for i in (1, 2, 100, 101):
        cur = _ngrams(ds.tokens_at(i).numpy())
        assert not (prev & cur), f"examples {i - 1} and {i} overlap"
        prev = cur


def test_pure_function_of_seed_and_index():
    a = SyntheticLmDataset(1000, 64, seed=3)
    b = SyntheticLmDataset(1000, 64, seed=3)
    c = SyntheticLmDataset(1000, 64, seed=4)
    assert (a.tokens_at(7) == b.tokens_at(7)).all()
    assert not (a.tokens_at(7) == c.tokens_at(7)).all()
    assert not (a.tokens_at(7) == a.tokens_at(8)).all()


def test_unigram_entropy_is_near_uniform():
    ds = SyntheticLmDataset(256, 8192, seed=0)
    toks = np.concatenate([ds.tokens_at(i).numpy() for i in range(8)])
    p = np.bincount(toks, minlength=256) / len(toks)
    h = -(p[p > 0] * np.log(p[p > 0])).sum()
    assert abs(h - math.log(256)) < 0.01
