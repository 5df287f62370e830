"""Pins oracle/quant.py: the known answers of the reference's own FP8 unit tests
(utilities/teeny-quant/src/quant/fp8.rs:270-357, groups per quant/groups.rs) and PyTorch's float8 casts."""
import numpy as np
import pytest
import torch

from oracle import quant as oq


def _rt(x, variant):
    return float(oq.f8_to_f32(oq.f32_to_f8(np.array([x], dtype=np.float32), variant), variant)[0])


@pytest.mark.parametrize("variant", [oq.E4M3, oq.E5M2])
def test_zero_and_signs_round_trip_exactly(variant):  # fp8.rs:284-293
    for x in (0.0, 1.0, -1.0, 2.0, -2.0):
        assert _rt(x, variant) == x


def test_reference_known_answers():
    assert _rt(448.0, oq.E4M3) == 448.0 and _rt(-448.0, oq.E4M3) == -448.0          # fp8.rs:296-299
    assert _rt(1.0e6, oq.E4M3) == 448.0 and _rt(np.inf, oq.E4M3) == 448.0           # fp8.rs:302-307 (saturates)
    assert _rt(57344.0, oq.E5M2) == 57344.0                                          # fp8.rs:310-312
    assert np.isinf(_rt(1.0e6, oq.E5M2))                                             # fp8.rs:315-318
    assert _rt(1.0e-10, oq.E4M3) == 0.0                                              # fp8.rs:321-325 (flushed)
    for variant in (oq.E4M3, oq.E5M2):                                               # fp8.rs:328-340
        for x in (0.1, 0.3, 1.5, 3.7, -12.25, 100.0):
            assert abs(x - _rt(x, variant)) < abs(x) * 0.2 + 0.01
    assert np.isnan(_rt(np.nan, oq.E4M3)) and np.isnan(_rt(np.nan, oq.E5M2))


def test_per_channel_uses_independent_scales():  # fp8.rs:343-356
    data = np.array([[0.1, -0.1], [200.0, -200.0]], dtype=np.float32)
    q, s = oq.quantize_fp8(data, "channel", axis=0)
    assert s.shape == (2,)
    back = oq.dequantize_fp8(q, s, "channel", axis=0)
    assert np.all(np.abs(data - back) < np.abs(data) * 0.3 + 0.01)
    assert np.allclose(s, np.array([0.1, 200.0], dtype=np.float32) / np.float32(448.0))
    assert np.array_equal(np.abs(oq.f8_to_f32(q)), np.full((2, 2), 448.0, dtype=np.float32))  # amax maps to 448


def test_group_ids_follow_the_reference_numbering():  # groups.rs:60-110
    g, n = oq.assign_groups((2, 6), "group", axis=1, group_size=4)
    assert n == 4 and g.tolist() == [[0, 0, 0, 0, 1, 1], [2, 2, 2, 2, 3, 3]]
    g, n = oq.assign_groups((2, 3), "channel", axis=0)
    assert n == 2 and g.tolist() == [[0, 0, 0], [1, 1, 1]]
    g, n = oq.assign_groups((2, 3), "channel", axis=1)
    assert n == 3 and g.tolist() == [[0, 1, 2], [0, 1, 2]]
    g, n = oq.assign_groups((2, 3), "tensor")
    assert n == 1 and not g.any()
    g, n = oq.assign_groups((2, 2, 4), "group", axis=2, group_size=2)  # other axes row-major, then the run
    assert n == 8 and g[1, 0].tolist() == [4, 4, 5, 5] and g[0, 1].tolist() == [2, 2, 3, 3]


@pytest.mark.parametrize("variant,dtype", [(oq.E4M3, torch.float8_e4m3fn), (oq.E5M2, torch.float8_e5m2)])
def test_decode_equals_pytorch_for_every_byte(variant, dtype):
    b = np.arange(256, dtype=np.uint8)
    ours = oq.f8_to_f32(b, variant)
    theirs = torch.from_numpy(b.copy()).view(dtype).float().numpy()
    assert np.array_equal(np.isnan(ours), np.isnan(theirs))
    ok = ~np.isnan(ours)
    assert np.array_equal(ours[ok], theirs[ok])
    assert np.array_equal(np.signbit(ours[ok]), np.signbit(theirs[ok]))


@pytest.mark.parametrize("variant,dtype,lo,hi", [(oq.E4M3, torch.float8_e4m3fn, 2.0 ** -6, 448.0),
                                                  (oq.E5M2, torch.float8_e5m2, 2.0 ** -14, 57344.0)])
def test_encode_equals_pytorch_on_the_normal_range(variant, dtype, lo, hi):
    """Round to nearest even, checked where the two definitions coincide: magnitudes from the smallest normal to the
    largest finite value (below, PyTorch rounds into subnormals and the reference flushes; above, they differ too)."""
    rng = np.random.default_rng(0)
    mag = np.exp(rng.uniform(np.log(lo), np.log(hi), 200000)).astype(np.float32)
    x = (mag * rng.choice([-1.0, 1.0], mag.size)).astype(np.float32)
    x = x[(np.abs(x) >= lo) & (np.abs(x) <= hi)]
    # exact ties and every representable value as well
    grid = oq.f8_to_f32(np.arange(256, dtype=np.uint8), variant)
    grid = grid[np.isfinite(grid) & (np.abs(grid) >= lo)]
    mids = ((grid[:-1].astype(np.float64) + grid[1:]) / 2).astype(np.float32)
    mids = mids[(np.abs(mids) >= lo) & (np.abs(mids) <= hi)]
    x = np.concatenate([x, grid, mids])
    ours = oq.f32_to_f8(x, variant)
    theirs = torch.from_numpy(x).to(dtype).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)


def test_quantize_dequantize_error_bound_and_linear_contract():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((96, 256)) * 0.05).astype(np.float32)
    for strategy, kw in (("tensor", {}), ("channel", {"axis": 0}), ("group", {"axis": 1, "group_size": 64})):
        q, s = oq.quantize_fp8(w, strategy, **kw)
        back = oq.dequantize_fp8(q, s, strategy, **kw)
        groups, _ = oq.assign_groups(w.shape, strategy, kw.get("axis"), kw.get("group_size"))
        # 3 mantissa bits: half an ulp is 2^-4 relative; values under the smallest normal (2^-6 * scale) go to zero
        bound = np.maximum(np.abs(w) * 2.0 ** -4, s[groups] * 2.0 ** -6)
        assert np.all(np.abs(back - w) <= bound * 1.0001)
        x = torch.randn(8, 256, generator=torch.Generator().manual_seed(2)).bfloat16().float().numpy()
        y = oq.linear_w8a16(x, q, s, strategy, **kw)
        assert np.allclose(y, x.astype(np.float64) @ back.astype(np.float64).T, rtol=1e-6, atol=1e-6)


# ---- integer schemes: the known answers of affine.rs:163-288 and pack4.rs:66-93 ----
def test_pack4_known_answers():
    values = np.arange(-8, 8, dtype=np.int8)
    packed = oq.pack_i4(values)
    assert packed.size == 8 and np.array_equal(oq.unpack_i4(packed, 16), values)     # pack4.rs:70-77
    odd = np.array([-8, 7, -1], dtype=np.int8)
    p = oq.pack_i4(odd)
    assert p.size == 2 and p.tolist() == [0x78, 0x0F] and np.array_equal(oq.unpack_i4(p, 3), odd)  # pack4.rs:80-86
    assert oq.pack_i4(np.array([], dtype=np.int8)).size == 0 and oq.unpack_i4(np.array([], dtype=np.uint8), 0).size == 0


def test_affine_ranges_and_round_trips():
    assert oq.qrange(8, True) == (-127, 127) and oq.qrange(8, False) == (-128, 127)  # affine.rs:46-51
    assert oq.qrange(4, True) == (-7, 7) and oq.qrange(4, False) == (-8, 7)
    data = np.array([-1.0, -0.5, 0.0, 0.5, 1.0], dtype=np.float32)
    q, s, zp = oq.quantize_affine(data, 8, True, "tensor")
    assert zp.tolist() == [0] and np.isclose(s[0], 1.0 / 127) and q.tolist() == [-127, -64, 0, 64, 127]  # halves away from zero
    assert np.abs(oq.dequantize_affine(q, s, zp, "tensor") - data).max() < 0.01
    pos = np.array([0.0, 1.0, 2.0, 3.0], dtype=np.float32)          # all-positive: asymmetric uses the whole range
    q, s, zp = oq.quantize_affine(pos, 8, False, "tensor")
    assert q.min() == -128 and q.max() == 127 and zp.tolist() == [-128] and np.isclose(s[0], 3.0 / 255)
    rows = np.array([[0.01, -0.01], [100.0, -100.0]], dtype=np.float32)
    q, s, zp = oq.quantize_affine(rows, 8, True, "channel", axis=0)
    assert np.allclose(s, [0.01 / 127, 100.0 / 127]) and np.abs(q).min() == 127
    q, _, _ = oq.quantize_affine(np.array([-10.0, 10.0], dtype=np.float32), 4, True, "tensor")
    assert q.tolist() == [-7, 7]                                      # affine.rs:280-287: clamped to the 4-bit range
    z, s, _ = oq.quantize_affine(np.zeros(4, dtype=np.float32), 8, True, "tensor")
    assert s.tolist() == [1.0] and not z.any()


def test_two_term_split_is_exact_within_ten_binades_of_the_row_maximum():
    """A bf16 value (8 significant bits) is the sum of two E4M3 numbers (4 bits each) while both stay normal."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(16, 512, generator=g) * torch.logspace(-2, 2, 16)[:, None]).bfloat16().float()
    x[3] = 0.0
    x[5, 7] = 0.0
    hi, lo, inv_s = oq.split_e4m3(x.numpy())
    back = (oq.f8_to_f32(hi).astype(np.float64) + oq.f8_to_f32(lo).astype(np.float64) / 16) * inv_s[:, None]
    amax = x.abs().amax(dim=1, keepdim=True).numpy()
    big = np.abs(x.numpy()) >= amax * 2.0 ** -10
    assert np.array_equal(back[big], x.numpy().astype(np.float64)[big])
    assert np.all(np.abs(back - x.numpy()) <= amax * 2.0 ** -17 + 1e-30)   # elsewhere: a small absolute error
    assert inv_s[3] == 1.0 and not hi[3].any() and not lo[3].any()
    scaled = np.abs(x.numpy()).max(axis=1) / inv_s
    assert np.all((scaled[scaled > 0] >= 128) & (scaled[scaled > 0] < 256))
