"""CPU restatement of the reference's FP8 weight quantiser (test infrastructure: only tests/, the smoke check and
bench.py's CPU leg may import this).

Follows utilities/teeny-quant/src/quant/fp8.rs and groups.rs of the reference:

  * ``f32_to_f8`` (fp8.rs:100-171): OCP FP8, round to nearest even at the target mantissa, magnitudes beyond the
    largest finite value saturate (E4M3: to 448, there is no infinity; E5M2: to infinity), anything below the smallest
    NORMAL of the target is flushed to (signed) zero, NaN -> exponent and mantissa all ones;
  * ``f8_to_f32`` (fp8.rs:175-206): full decode, subnormals and NaN / infinity included;
  * ``assign_groups`` (groups.rs:84-110): "tensor" = one group; "channel" with axis a = group id is the index along a;
    "group" with (axis, size) = contiguous runs of `size` along the axis, every combination of the other axes its own
    set (ids: other axes row-major, then the run index);
  * ``quantize_fp8`` (fp8.rs:224-259): scale = amax / max_finite (1.0 for an all-zero group), q = f32_to_f8(x / scale);
  * ``dequantize_fp8`` (fp8.rs:262-268): f8_to_f32(q) * scale;
  * ``linear_w8a16``: what a weight-only GEMM over such a tensor has to produce: bf16 activations times the
    dequantised f32 weight, accumulated in float32 (float64 here), rounded once to bf16.  The reference has no such
    kernel; this states the contract of include/teeny_b200.h's teeny_linear_w8a16_forward.

Pinned by tests/test_oracle_quant.py against every known-answer case of fp8.rs's own unit tests (fp8.rs:270-357), and
against PyTorch's float8_e4m3fn / float8_e5m2 casts: decode for all 256 bytes of both formats, encode on the values
where the two definitions agree (PyTorch keeps subnormal results, the reference flushes them; PyTorch's E4M3 cast of an
out-of-range value gives NaN, the reference saturates).
"""
import numpy as np

E4M3, E5M2 = "e4m3", "e5m2"
_FMT = {  # mantissa bits, exponent bits, bias, largest finite unbiased exponent, largest finite value, has infinity
    E4M3: (3, 4, 7, 8, 448.0, False),
    E5M2: (2, 5, 15, 15, 57344.0, True),
}


def f32_to_f8(x, variant=E4M3):
    """Array of float32 -> array of uint8 (fp8.rs:100-171)."""
    m_bits, e_bits, bias, max_unb, _, has_inf = _FMT[variant]
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.int64)
    sign = ((bits >> 31) & 1).astype(np.int64)
    exp_mask = (1 << e_bits) - 1
    sat = (sign << 7) | (exp_mask << m_bits) | (0 if has_inf else ((1 << m_bits) - 2))
    unb = ((bits >> 23) & 0xFF) - 127
    sig = (1 << 23) | (bits & 0x7FFFFF)
    shift = 23 - m_bits
    half, mask = 1 << (shift - 1), (1 << shift) - 1
    rem = sig & mask
    rounded = sig >> shift
    rounded = rounded + ((rem > half) | ((rem == half) & ((rounded & 1) == 1)))
    implicit = 1 << m_bits
    carry = rounded == (implicit << 1)
    rounded = np.where(carry, implicit, rounded)
    exp_out = unb + carry
    normal = (sign << 7) | ((exp_out + bias) << m_bits) | (rounded - implicit)
    out = np.where(exp_out > max_unb, sat, normal)
    out = np.where(unb > max_unb, sat, out)
    out = np.where(unb < 1 - bias, sign << 7, out)       # below the smallest normal: flushed
    out = np.where(np.isinf(x), sat, out)
    out = np.where(np.isnan(x), (sign << 7) | (exp_mask << m_bits) | ((1 << m_bits) - 1), out)
    out = np.where(x == 0.0, sign << 7, out)
    return out.astype(np.uint8)


def f8_to_f32(b, variant=E4M3):
    """Array of uint8 -> array of float32 (fp8.rs:175-206)."""
    m_bits, e_bits, bias, _, _, _ = _FMT[variant]
    b = np.asarray(b, dtype=np.uint8).astype(np.int64)
    sign = np.where((b >> 7) & 1, -1.0, 1.0)
    e = (b >> m_bits) & ((1 << e_bits) - 1)
    m = b & ((1 << m_bits) - 1)
    frac = m / float(1 << m_bits)
    val = np.where(e == 0, frac * 2.0 ** (1 - bias), (1.0 + frac) * np.exp2((e - bias).astype(np.float64)))
    val = sign * val
    all_ones = e == (1 << e_bits) - 1
    if variant == E4M3:
        val = np.where(all_ones & (m == (1 << m_bits) - 1), np.nan, val)
    else:
        val = np.where(all_ones, np.where(m == 0, sign * np.inf, np.nan), val)
    return val.astype(np.float32)


def assign_groups(shape, strategy, axis=None, group_size=None):
    """(flat group id per element as an array of `shape`, number of groups) -- groups.rs:84-110."""
    shape = tuple(int(s) for s in shape)
    if strategy == "tensor":
        return np.zeros(shape, dtype=np.int64), 1
    idx = np.indices(shape)
    if strategy == "channel":
        return idx[axis].astype(np.int64), shape[axis]
    if strategy != "group":
        raise ValueError(strategy)
    outer, mult = np.zeros(shape, dtype=np.int64), 1
    for d in reversed(range(len(shape))):
        if d == axis:
            continue
        outer += idx[d] * mult
        mult *= shape[d]
    along = -(-shape[axis] // group_size)
    return outer * along + idx[axis] // group_size, mult * along


def quantize_fp8(w, strategy="channel", axis=0, group_size=None, variant=E4M3):
    """(bytes of w's shape, float32 scales [groups]) -- fp8.rs:224-259."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    groups, n = assign_groups(w.shape, strategy, axis, group_size)
    amax = np.zeros(n, dtype=np.float32)
    np.maximum.at(amax, groups.ravel(), np.abs(w).ravel())
    scales = np.where(amax == 0.0, np.float32(1.0), amax / np.float32(_FMT[variant][4])).astype(np.float32)
    return f32_to_f8((w / scales[groups]).astype(np.float32), variant), scales


def dequantize_fp8(q, scales, strategy="channel", axis=0, group_size=None, variant=E4M3):
    """float32 array of q's shape -- fp8.rs:262-268."""
    groups, _ = assign_groups(q.shape, strategy, axis, group_size)
    return (f8_to_f32(q, variant) * np.asarray(scales, dtype=np.float32)[groups]).astype(np.float32)


def linear_w8a16(x_bf16_as_f32, q, scales, strategy="channel", axis=0, group_size=None, bias=None):
    """y = x @ dequantize(q)^T (+ bias), float64 accumulation; the caller rounds to bf16.  x: [M, K] float32 holding
    bf16 values; q: [N, K] uint8."""
    w = dequantize_fp8(q, scales, strategy, axis, group_size).astype(np.float64)
    y = np.asarray(x_bf16_as_f32, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y.astype(np.float32)
