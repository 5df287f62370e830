"""Collect the reference's own golden vectors for the GEMM / attention / Qwen3-forward hot path.

The reference keeps flat little-endian f32 ``.bin`` fixtures under
``kernels/teeny-kernels/tests/fixtures/<op>/`` (written by PyTorch with ``torch.manual_seed(42)``,
``kernels/teeny-kernels/tests/fixtures/generate.py:16``).  This script packs the ones that pin the
hot path into one ``reference_fixtures.npz`` (shapes restored from the constants in generate.py) so
the tests can run on machines that do not have the reference checkout.

It also records the inline ramp case of ``kernels/teeny-kernels/tests/test_gemm.rs:107-120``
(``matmul_forward`` has no ``.bin`` fixture: the test derives A, B and the expectation from
``i / (m*k)`` ramps and a naive f32 triple loop), regenerated here with the same arithmetic.

Run once where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/teenygrad
"""
import os
import sys

import numpy as np


def _load(base, op, name, shape):
    a = np.fromfile(os.path.join(base, op, name + ".bin"), dtype="<f4")
    return a.reshape(shape)


def main(ref_root):
    base = os.path.join(ref_root, "kernels", "teeny-kernels", "tests", "fixtures")
    out = {}
    # linear: M=64, N=48, K=64 (generate.py:75-91; test_linear.rs)
    out["linear_input"] = _load(base, "linear", "input", (64, 64))
    out["linear_weight"] = _load(base, "linear", "weight", (48, 64))
    out["linear_bias"] = _load(base, "linear", "bias", (48,))
    out["linear_expected_no_bias"] = _load(base, "linear", "expected_no_bias", (64, 48))
    out["linear_expected_with_bias"] = _load(base, "linear", "expected_with_bias", (64, 48))
    # flash_attn2: BH=4, N_CTX=8, D=64, scale=1/8, non-causal (generate.py:701-727)
    for n in ("q", "k", "v", "expected_forward_o"):
        out["fa2_" + n] = _load(base, "flash_attn2", n, (4, 8, 64))
    out["fa2_expected_forward_l"] = _load(base, "flash_attn2", "expected_forward_l", (4, 8))
    # rmsnorm: 16x128, eps 1e-8 (generate.py:541-556)
    out["rmsnorm_x"] = _load(base, "rmsnorm", "x", (16, 128))
    out["rmsnorm_weight"] = _load(base, "rmsnorm", "weight", (128,))
    out["rmsnorm_expected_forward"] = _load(base, "rmsnorm", "expected_forward", (16, 128))
    out["rmsnorm_expected_rrms"] = _load(base, "rmsnorm", "expected_rrms", (16,))
    # silu: 1024 (generate.py:458-459)
    out["silu_x"] = _load(base, "silu", "x", (1024,))
    out["silu_expected_forward"] = _load(base, "silu", "expected_forward", (1024,))
    # elemwise_binary: 1024 (generate.py:890-898)
    for n in ("a", "b", "expected_mul", "expected_sum"):
        out["binary_" + n] = _load(base, "elemwise_binary", n, (1024,))
    # elemwise_add: 1024 (fixtures/elemwise_add/generate.py:37-43)
    for n in ("a", "b", "expected_fwd"):
        out["add_" + n] = _load(base, "elemwise_add", n, (1024,))
    # softmax: 64x128
    out["softmax_x_forward"] = _load(base, "softmax", "x_forward", (64, 128))
    out["softmax_expected_forward"] = _load(base, "softmax", "expected_forward", (64, 128))

    # matmul_forward ramp case (test_gemm.rs:107-120): m=64, n=48, k=64, f32 sequential accumulation.
    m, n, k = 64, 48, 64
    a = (np.arange(m * k, dtype=np.float32) / np.float32(m * k)).astype(np.float32).reshape(m, k)
    b = (np.arange(k * n, dtype=np.float32) / np.float32(k * n)).astype(np.float32).reshape(k, n)
    c = np.zeros((m, n), dtype=np.float32)
    for ki in range(k):  # same summation order as the test's inner loop, vectorised over (mi, ni)
        c = (c + a[:, ki:ki + 1] * b[ki:ki + 1, :]).astype(np.float32)
    out["gemm_ramp_a"], out["gemm_ramp_b"], out["gemm_ramp_expected"] = a, b, c

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1])
