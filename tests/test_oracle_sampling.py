"""The sampling oracle against facts that hold by definition (no GPU)."""
import numpy as np

from oracle import sampling as osamp


def _row(seed, n=4096):
    rng = np.random.default_rng(seed)
    # bf16-like coarse values, so ties occur as they do in real logits
    return (np.round(rng.normal(0, 3, n) * 16) / 16).astype(np.float32)


def test_top_k_one_is_argmax_with_lowest_index_on_ties():
    row = _row(0)
    row[[100, 7, 3000]] = row.max() + 1
    idx, prob, c, n, cand = osamp.sample_row(row, 0.7, 1, 1.0, 0.99)
    assert idx == 7 and n == 1 and abs(prob - 1.0) < 1e-6


def test_candidates_order_value_desc_then_index_asc():
    row = _row(1)
    cand = osamp.candidates(row, 50)
    vals = row[cand]
    assert np.all(vals[:-1] >= vals[1:])
    same = vals[:-1] == vals[1:]
    assert np.all(cand[:-1][same] < cand[1:][same])
    # nothing outside beats the weakest candidate
    rest = np.setdiff1d(np.arange(row.size), cand)
    assert row[rest].max() <= vals[-1]


def test_nucleus_is_the_shortest_prefix_reaching_top_p():
    row = _row(2)
    idx, prob, c, n, cand = osamp.sample_row(row, 1.0, 200, 0.9, 0.5)
    assert c[n - 1] >= np.float32(0.9) * c[-1] and (n == 1 or c[n - 2] < np.float32(0.9) * c[-1])
    assert idx in cand[:n]


def test_u_sweeps_the_cdf_monotonically():
    row = _row(3)
    picks = [osamp.sample_row(row, 1.3, 64, 0.95, u)[0] for u in np.linspace(0, 0.999, 200)]
    cand = list(osamp.candidates(row, 64))
    ranks = [cand.index(p) for p in picks]
    assert ranks[0] == 0 and all(a <= b for a, b in zip(ranks, ranks[1:]))


def test_empirical_frequencies_follow_the_probabilities():
    row = _row(4, 512)
    rng = np.random.default_rng(5)
    us = rng.random(20000).astype(np.float32)
    picks = np.array([osamp.sample_row(row, 1.0, 8, 1.0, u)[0] for u in us])
    cand = osamp.candidates(row, 8)
    p = np.exp(row[cand] - row[cand][0]); p /= p.sum()
    freq = np.array([(picks == c).mean() for c in cand])
    assert np.abs(freq - p).max() < 0.015
