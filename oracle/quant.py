"""CPU restatement of the reference's weight quantiser, FP8 and integer schemes (test infrastructure: only tests/, the
smoke check and bench.py's CPU leg may import this).

Follows utilities/teeny-quant/src/quant/fp8.rs, groups.rs, affine.rs and pack4.rs of the reference (the integer
functions cite their lines where they stand, at the end of the file):

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

Pinned by tests/test_oracle_quant.py against every known-answer case of fp8.rs's own unit tests (fp8.rs:270-357), of
affine.rs:163-288 and of pack4.rs:66-93, and
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


# ---- integer schemes: utilities/teeny-quant/src/quant/affine.rs and pack4.rs ----
def _round_half_away(x):
    """Rust's f32::round: halves away from zero."""
    return np.sign(x) * np.floor(np.abs(x) + np.float32(0.5))


def qrange(bits, symmetric):
    """affine.rs:46-51: 8 bits -> [-127, 127] symmetric, [-128, 127] asymmetric; 4 bits -> [-7, 7] / [-8, 7]."""
    qmax = (1 << (bits - 1)) - 1
    return (-qmax if symmetric else -qmax - 1), qmax


def quantize_affine(w, bits=8, symmetric=True, strategy="channel", axis=0, group_size=None):
    """(int8 values of w's shape, float32 scales [groups], int32 zero points [groups]) -- affine.rs:55-148: per group
    lo = min(min x, 0), hi = max(max x, 0); symmetric: scale = max(|lo|, |hi|) / qmax (1 if 0), zero point 0;
    asymmetric: scale = (hi - lo) / (qmax - qmin) (1 if hi == lo), zero point = round(qmin - lo / scale) clamped;
    q = clamp(round(x / scale) + zero point)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    qmin, qmax = qrange(bits, symmetric)
    groups, n = assign_groups(w.shape, strategy, axis, group_size)
    lo = np.full(n, np.inf, dtype=np.float32)
    hi = np.full(n, -np.inf, dtype=np.float32)
    np.minimum.at(lo, groups.ravel(), w.ravel())
    np.maximum.at(hi, groups.ravel(), w.ravel())
    lo, hi = np.minimum(lo, np.float32(0)), np.maximum(hi, np.float32(0))
    if symmetric:
        amax = np.maximum(np.abs(lo), np.abs(hi))
        scale = np.where(amax == 0, np.float32(1), amax / np.float32(qmax)).astype(np.float32)
        zp = np.zeros(n, dtype=np.int32)
    else:
        scale = np.where(hi == lo, np.float32(1), (hi - lo) / np.float32(qmax - qmin)).astype(np.float32)
        zp = np.clip(_round_half_away(np.float32(qmin) - lo / scale).astype(np.int64), qmin, qmax).astype(np.int32)
    q = _round_half_away((w / scale[groups]).astype(np.float32)).astype(np.int64) + zp[groups]
    return np.clip(q, qmin, qmax).astype(np.int8), scale, zp


def dequantize_affine(q, scales, zero_points=None, strategy="channel", axis=0, group_size=None):
    """float32 (q - zero point) * scale -- affine.rs:151-161."""
    groups, _ = assign_groups(q.shape, strategy, axis, group_size)
    zp = np.zeros(len(scales), dtype=np.int32) if zero_points is None else np.asarray(zero_points, dtype=np.int32)
    return ((q.astype(np.int32) - zp[groups]).astype(np.float32) * np.asarray(scales, dtype=np.float32)[groups])


def pack_i4(values):
    """pack4.rs:31-40: two consecutive elements (row-major, flattened) per byte, the first in the low nibble; an odd
    count leaves the last high nibble zero."""
    v = np.asarray(values, dtype=np.int8).ravel().astype(np.uint8) & 0x0F
    if v.size % 2:
        v = np.concatenate([v, np.zeros(1, dtype=np.uint8)])
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)


def unpack_i4(packed, n):
    """pack4.rs:43-64: n sign-extended nibbles."""
    b = np.asarray(packed, dtype=np.uint8)
    nib = np.stack([b & 0x0F, b >> 4], axis=1).ravel()[:n].astype(np.int16)
    return np.where(nib >= 8, nib - 16, nib).astype(np.int8)


# ---- two-term FP8 activations (the F8 variant of the weight-only GEMM; not part of the reference) ----
def split_e4m3(x_bf16_as_f32):
    """(hi, lo16, inv_s): per row s = 2^(7 - floor(log2 max|x|)) (1 for an all-zero row), hi = e4m3(x s), lo16 =
    e4m3((x s - hi) 16), both round to nearest even with subnormals kept (PyTorch's float8_e4m3fn cast, which
    tests/test_oracle_quant.py holds f8_to_f32 to for all 256 bytes); the value represented is (hi + lo16 / 16) inv_s."""
    import torch
    x = torch.as_tensor(np.asarray(x_bf16_as_f32, dtype=np.float32))
    amax = x.abs().amax(dim=1)
    e = torch.floor(torch.log2(torch.where(amax > 0, amax, torch.ones_like(amax))))
    p = torch.where(amax > 0, (7 - e).clamp(-100, 100), torch.zeros_like(e))
    s = torch.pow(torch.tensor(2.0, dtype=torch.float64), p.double()).float()[:, None]
    xs = x * s
    hi = xs.to(torch.float8_e4m3fn)
    lo = ((xs - hi.float()) * 16.0).to(torch.float8_e4m3fn)
    return hi.view(torch.uint8).numpy(), lo.view(torch.uint8).numpy(), (1.0 / s[:, 0]).numpy()


def linear_w8a8x2(hi, lo16, inv_s, q, scales, strategy="channel", axis=0, bias=None):
    """y = inv_s * ((hi + lo16 / 16) @ dequantize(q)^T) (+ bias) in float64; the caller rounds to bf16."""
    x = (f8_to_f32(hi).astype(np.float64) + f8_to_f32(lo16).astype(np.float64) / 16.0) * np.asarray(inv_s, dtype=np.float64)[:, None]
    y = x @ dequantize_fp8(q, scales, strategy, axis).astype(np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y.astype(np.float32)
