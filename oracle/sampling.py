"""CPU restatement of the sampling step behind the LM head (test infrastructure: only tests/ may import this).

The reference ships the row softmax next to the logits (kernels/teeny-kernels/src/nn/activation/softmax.rs:39-69) and
leaves Op::TopK unlowered (kernels/teeny-kernels/src/graph/mod.rs:2784); temperature / top-k / top-p follow the usual
logits-processor definitions, pinned here so the CUDA kernel has something exact to be compared with:

  1. candidates = the top_k entries of the row by (logit descending, index ascending);
  2. e_i = exp((l_i - l_0) / temperature) in float32, c_i = e_0 + ... + e_i summed sequentially in float32;
  3. nucleus = the shortest prefix with c_{n-1} >= top_p * c_last (at least one candidate);
  4. sample = the first candidate i < n with c_i > u * c_{n-1}.
The reference has no sampler to pin this against; it is pinned instead to the logits processors of ``transformers``
(the package the reference's Qwen3 script generates with, support/teeny-torch/python/tests/test_qwen3.py:18):
tests/test_oracle_sampling.py checks that the candidate set equals TopKLogitsWarper's kept set, the nucleus equals what
TopPLogitsWarper keeps after it, and the in-nucleus probabilities equal the softmax of the surviving scores (one
stated difference: on a tie at the k-th value the warper keeps every tied entry, this keeps exactly k, lowest indices
first).  The softmax part is also pinned by the reference's own softmax fixture through oracle/cpu.py.
"""
import numpy as np


def candidates(row_f32, top_k):
    """Indices of the top_k entries by (value descending, index ascending)."""
    order = np.lexsort((np.arange(row_f32.size), -row_f32.astype(np.float64)))
    return order[:min(top_k, row_f32.size)]


def sample_row(row_f32, temperature, top_k, top_p, u):
    """Returns (index, probability inside the nucleus, cumulative masses c, nucleus length n, candidate indices)."""
    cand = candidates(row_f32, top_k)
    l = row_f32[cand].astype(np.float32)
    inv_t = np.float32(1.0) / np.float32(temperature)
    e = np.exp((l - l[0]) * inv_t).astype(np.float32)
    c = np.cumsum(e, dtype=np.float32)  # sequential float32 sums
    want = np.float32(top_p) * c[-1]
    n = int(np.argmax(c >= want)) + 1 if np.any(c >= want) else len(c)
    target = np.float32(u) * c[n - 1]
    hit = np.nonzero(c[:n] > target)[0]
    i = int(hit[0]) if hit.size else n - 1
    return int(cand[i]), float(e[i] / c[n - 1]), c, n, cand


def sample(logits_f32, temperature, top_k, top_p, u):
    return np.array([sample_row(logits_f32[r], temperature, top_k, top_p, u[r])[0] for r in range(logits_f32.shape[0])],
                    dtype=np.int32)


def uniform(seed, step, row):
    """u in [0, 1) for token `step` of a generation and batch row `row`: the runner's stateless hash
    (teenygrad_b200/csrc/sampling.cu, sampling_uniform_kernel), restated on Python integers."""
    m = (1 << 64) - 1
    x = (seed ^ (step * 0x9E3779B97F4A7C15) ^ (row * 0xBF58476D1CE4E5B9)) & m
    x ^= x >> 30; x = (x * 0xBF58476D1CE4E5B9) & m
    x ^= x >> 27; x = (x * 0x94D049BB133111EB) & m
    x ^= x >> 31
    return np.float32(x >> 40) * np.float32(1.0 / 16777216.0)
