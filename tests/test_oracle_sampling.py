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


def test_candidate_set_nucleus_and_probabilities_match_transformers_warpers():
    """Pins the oracle to the logits processors of ``transformers`` (the package the reference's Qwen3 script
    generates with): temperature, then TopKLogitsWarper, then TopPLogitsWarper.  On rows without a tie at the k-th
    value the oracle's candidate set is the warper's kept set, its nucleus is what survives top-p, and its in-nucleus
    probabilities are the softmax of the surviving scores.  (With ties at the k-th value the warper keeps every tied
    entry, i.e. more than k; the oracle and the kernel keep exactly k, lowest indices first.)"""
    import torch
    from transformers.generation.logits_process import TemperatureLogitsWarper, TopKLogitsWarper, TopPLogitsWarper
    rng = np.random.default_rng(11)
    for (n, temperature, top_k, top_p) in [(4096, 0.8, 50, 0.9), (151936, 1.5, 1024, 0.95), (777, 0.3, 64, 0.5),
                                           (32000, 1.0, 40, 1.0), (5000, 0.7, 1, 0.9)]:
        row = rng.normal(0, 3, n).astype(np.float32)
        scores = torch.from_numpy(row)[None]
        ids = torch.zeros(1, 1, dtype=torch.long)
        s = TemperatureLogitsWarper(float(temperature))(ids, scores)
        s_k = TopKLogitsWarper(top_k=top_k)(ids, s)
        s_p = TopPLogitsWarper(top_p=float(top_p))(ids, s_k) if top_p < 1.0 else s_k
        kept_k = set(torch.nonzero(torch.isfinite(s_k[0]))[:, 0].tolist())
        kept_p = set(torch.nonzero(torch.isfinite(s_p[0]))[:, 0].tolist())
        probs = torch.softmax(s_p[0], dim=-1).numpy()
        _, _, c, nuc, cand = osamp.sample_row(row, temperature, top_k, top_p, 0.5)
        assert set(cand.tolist()) == kept_k
        assert set(cand[:nuc].tolist()) == kept_p, (n, nuc, len(kept_p))
        for u in (0.0, 0.3, 0.77, 0.999):
            idx, prob, _, _, _ = osamp.sample_row(row, temperature, top_k, top_p, u)
            assert idx in kept_p
            assert abs(prob - probs[idx]) < 2e-5 * max(1.0, probs[idx] * 1e3)
        # and the pick is the inverse CDF over the warper's distribution taken in (probability desc) order
        order = cand[:nuc]
        cdf = np.cumsum(probs[order].astype(np.float64))
        for u in (0.05, 0.5, 0.93):
            idx = osamp.sample_row(row, temperature, top_k, top_p, u)[0]
            j = list(order).index(idx)
            lo = cdf[j - 1] if j else 0.0
            assert lo - 1e-5 <= u <= cdf[j] + 1e-5
