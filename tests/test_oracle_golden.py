"""Pins the CPU oracle against every golden vector the reference's tests hold for the hot path.

Tolerances are the reference's own (kernels/teeny-kernels/tests): linear 1e-1 + 2e-2*|e| is its GPU/TF32
bound -- the f32 oracle is held to a much tighter 1e-4 relative-to-scale bound here; FA2 O and L < 1e-4;
RMSNorm y and rrms < 1e-4; SiLU < 1e-5; add exact.
"""
import numpy as np

from oracle import cpu as oc


def _scaled_err(a, e):
    return float(np.abs(a - e).max() / max(np.abs(e).max(), 1e-30))


def test_matmul_ramp_case(golden):
    c = oc.matmul_f32(golden["gemm_ramp_a"], golden["gemm_ramp_b"])
    assert np.array_equal(c, golden["gemm_ramp_expected"])  # same f32 summation order -> bit exact


def test_linear_fixture(golden):
    y = oc.linear_f32(golden["linear_input"], golden["linear_weight"])
    assert _scaled_err(y, golden["linear_expected_no_bias"]) < 1e-6
    yb = oc.linear_f32(golden["linear_input"], golden["linear_weight"], golden["linear_bias"])
    assert _scaled_err(yb, golden["linear_expected_with_bias"]) < 1e-6
    e = golden["linear_expected_with_bias"]
    assert np.all(np.abs(yb - e) < 1e-1 + 2e-2 * np.abs(e))  # reference bound, test_linear.rs:42-47


def test_flash_attn2_fixture(golden):
    q, k, v = (golden["fa2_" + n][None] for n in ("q", "k", "v"))  # [1, BH, N_CTX, D]
    o, lse = oc.attention_f32(q, k, v, scale=0.125, causal=False)
    assert np.abs(o[0] - golden["fa2_expected_forward_o"]).max() < 1e-4   # test_flash_attn2.rs:152-168
    assert np.abs(lse[0] - golden["fa2_expected_forward_l"]).max() < 1e-4


def test_rmsnorm_fixture(golden):
    y, rrms = oc.rms_norm_f32(golden["rmsnorm_x"], golden["rmsnorm_weight"], 1e-8)
    assert np.abs(y - golden["rmsnorm_expected_forward"]).max() < 1e-4    # test_rmsnorm.rs:142-151
    assert np.abs(rrms - golden["rmsnorm_expected_rrms"]).max() < 1e-4


def test_silu_fixture(golden):
    assert np.abs(oc.silu_f32(golden["silu_x"]) - golden["silu_expected_forward"]).max() < 1e-5


def test_mul_add_fixtures(golden):
    assert np.array_equal(oc.mul_f32(golden["binary_a"], golden["binary_b"]), golden["binary_expected_mul"])
    assert np.array_equal(oc.add_f32(golden["binary_a"], golden["binary_b"]), golden["binary_expected_sum"])
    assert np.array_equal(oc.add_f32(golden["add_a"], golden["add_b"]), golden["add_expected_fwd"])


def test_softmax_fixture(golden):
    y = oc.softmax_f32(golden["softmax_x_forward"])
    assert np.abs(y - golden["softmax_expected_forward"]).max() < 1e-6


def test_attention_gqa_causal_matches_torch():
    """The GQA + causal extension of the oracle agrees with PyTorch SDPA semantics (repeat KV heads, mask)."""
    import torch
    g = torch.Generator().manual_seed(2)
    B, Hq, Hkv, Sq, Skv, D = 2, 4, 2, 5, 9, 16
    q = torch.randn(B, Hq, Sq, D, generator=g)
    k = torch.randn(B, Hkv, Skv, D, generator=g)
    v = torch.randn(B, Hkv, Skv, D, generator=g)
    o, lse = oc.attention_f32(q.numpy(), k.numpy(), v.numpy(), D ** -0.5, causal=True)
    ke, ve = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    mask = torch.arange(Skv)[None, :] <= (torch.arange(Sq)[:, None] + (Skv - Sq))
    ref = torch.nn.functional.scaled_dot_product_attention(q, ke, ve, attn_mask=mask, scale=D ** -0.5)
    assert np.abs(o - ref.numpy()).max() < 1e-5
    ob, lb = oc.attention_bf16(q.bfloat16(), k.bfloat16(), v.bfloat16(), D ** -0.5, causal=True)
    assert (ob.float() - ref).abs().max() < 5e-2
