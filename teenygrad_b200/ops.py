"""Operator wrappers over torch CUDA tensors: argument checks, then one C-ABI call on torch's current stream.

Names follow the reference's kernels (matmul_forward, linear_forward, flash_attention2_forward,
rms_norm_forward, silu_forward, elemwise_mul_forward, elemwise_add_forward, softmax_forward) plus the fused
Qwen3-layer kernels.  Nothing here computes: a missing library or a non-zero status raises.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import lib, check, AttnShape

_BF16, _F32 = torch.bfloat16, torch.float32


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _req(t, dtype=None, name="tensor"):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    return t


def _sfx(t):
    if t.dtype == _F32:
        return "f32"
    if t.dtype == _BF16:
        return "bf16"
    raise ValueError(f"unsupported dtype {t.dtype}")


def device_error(clear=True):
    """Synchronise and return the device error word (0 = no kernel gave up on a wait)."""
    return lib.teeny_device_error(1 if clear else 0)


def gemm_scratch(M, N, K, device="cuda"):
    """Zero-filled split-K scratch for linear_forward at this shape (None when the shape never splits)."""
    n = lib.teeny_gemm_scratch_bytes(M, N, K)
    return torch.zeros(n, dtype=torch.uint8, device=device) if n else None


def matmul_f32_scratch(M, N, K, device="cuda"):
    """Scratch that sends the f32 matmul to the tensor cores (operands split into bf16 terms); without it the f32
    entry point runs on the CUDA cores."""
    return torch.empty(lib.teeny_matmul_f32_scratch_bytes(M, N, K), dtype=torch.uint8, device=device)


def matmul_forward(a, b, out=None, scratch=None):
    """C = A @ B, row-major [M,K] x [K,N]."""
    _req(a, name="a"); _req(b, a.dtype, "b")
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[1]
    out = torch.empty(M, N, dtype=a.dtype, device=a.device) if out is None else out
    fn = getattr(lib, f"matmul_forward_entry_point_{_sfx(a)}")
    check(fn(_ptr(a), _ptr(b), _ptr(out), M, N, K, _ptr(scratch), scratch.numel() if scratch is not None else 0,
             _stream()), "matmul_forward")
    return out


def linear_forward(x, w, bias=None, out=None, scratch=None):
    """Y = X @ W^T (+ bias); x [M,K] and w [N,K] may be strided 2-D views."""
    _req(x, name="x"); _req(w, x.dtype, "w")
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty(M, N, dtype=x.dtype, device=x.device) if out is None else out
    fn = getattr(lib, f"linear_forward_entry_point_{_sfx(x)}")
    check(fn(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, x.stride(0), x.stride(1), w.stride(0), w.stride(1),
             out.stride(0), out.stride(1), _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()),
          "linear_forward")
    return out


def flash_attention2_forward(q, k, v, softmax_scale, want_lse=True):
    """Reference layout [BH, n_ctx, D], non-causal.  Returns (o, l)."""
    _req(q, name="q")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    BH, nq, D = q.shape
    nk = k.shape[1]
    o = torch.empty_like(q)
    l = torch.empty(BH, nq, dtype=_F32, device=q.device) if want_lse else None
    fn = getattr(lib, f"flash_attention2_forward_entry_point_{_sfx(q)}")
    check(fn(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(l), nq, nk, float(softmax_scale), float("-inf"), BH, D,
             _stream()), "flash_attention2_forward")
    return o, l


def _shape_of(q, k, v, o, scale, causal):
    """q/o [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] as (possibly strided) views with unit stride on D."""
    for t in (q, k, v, o):
        if t.stride(-1) != 1:
            raise ValueError("head_dim must be contiguous")
    B, Hq, Sq, D = q.shape
    s = AttnShape()
    s.B, s.Hq, s.Hkv, s.Sq, s.Skv, s.D = B, Hq, k.shape[1], Sq, k.shape[2], D
    s.q_sb, s.q_sh, s.q_ss = q.stride(0), q.stride(1), q.stride(2)
    s.k_sb, s.k_sh, s.k_ss = k.stride(0), k.stride(1), k.stride(2)
    s.v_sb, s.v_sh, s.v_ss = v.stride(0), v.stride(1), v.stride(2)
    s.o_sb, s.o_sh, s.o_ss = o.stride(0), o.stride(1), o.stride(2)
    s.scale, s.causal = float(scale), int(bool(causal))
    return s


def flash_attn_fwd(q, k, v, scale, causal=True, out=None, want_lse=False):
    """Causal grouped-query attention, bf16; q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] views."""
    _req(q, _BF16, "q"); _req(k, _BF16, "k"); _req(v, _BF16, "v")
    o = torch.empty(q.shape, dtype=_BF16, device=q.device) if out is None else out
    lse = torch.empty(q.shape[:3], dtype=_F32, device=q.device) if want_lse else None
    s = _shape_of(q, k, v, o, scale, causal)
    check(lib.teeny_flash_attn_fwd_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), C.byref(s), _stream()),
          "flash_attn_fwd")
    return (o, lse) if want_lse else o


def flash_attn_decode(q, k_cache, v_cache, kv_len, scale, out=None, scratch=None):
    """q [B,Hq,1,D]; caches [B,Hkv,cap,D]; kv_len an int or a 1-element int32 CUDA tensor."""
    _req(q, _BF16, "q")
    o = torch.empty(q.shape, dtype=_BF16, device=q.device) if out is None else out
    s = _shape_of(q, k_cache, v_cache, o, scale, False)
    need = lib.teeny_attn_decode_scratch_bytes(s.B, s.Hq, s.D, s.Skv)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    dev_len = kv_len if torch.is_tensor(kv_len) else None
    check(lib.teeny_flash_attn_decode_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(o), C.byref(s),
                                           0 if dev_len is not None else int(kv_len), _ptr(dev_len), _ptr(scratch),
                                           scratch.numel(), _stream()), "flash_attn_decode")
    return o


def rms_norm_forward(x, weight, eps, want_rrms=False):
    _req(x, name="x"); _req(weight, x.dtype, "weight")
    x = x.contiguous()
    M, N = x.shape
    y = torch.empty_like(x)
    rrms = torch.empty(M, dtype=_F32, device=x.device) if want_rrms else None
    fn = getattr(lib, f"rms_norm_forward_entry_point_{_sfx(x)}")
    check(fn(_ptr(x), _ptr(y), _ptr(weight), _ptr(rrms), M, N, float(eps), _stream()), "rms_norm_forward")
    return (y, rrms) if want_rrms else y


def _flat(name, a, b=None):
    _req(a, name="a")
    a = a.contiguous()
    out = torch.empty_like(a)
    fn = getattr(lib, f"{name}_entry_point_{_sfx(a)}")
    if b is None:
        check(fn(_ptr(a), _ptr(out), a.numel(), _stream()), name)
    else:
        b = _req(b, a.dtype, "b").contiguous()
        check(fn(_ptr(a), _ptr(b), _ptr(out), a.numel(), _stream()), name)
    return out


def silu_forward(x):
    return _flat("silu_forward", x)


def elemwise_mul_forward(a, b):
    return _flat("elemwise_mul_forward", a, b)


def elemwise_add_forward(a, b):
    return _flat("elemwise_add_forward", a, b)


def softmax_forward(x):
    _req(x, name="x")
    x = x.contiguous()
    y = torch.empty_like(x)
    fn = getattr(lib, f"softmax_forward_entry_point_{_sfx(x)}")
    check(fn(_ptr(x), _ptr(y), x.shape[0], x.shape[1], _stream()), "softmax_forward")
    return y


def add_rms_norm(x, residual, weight, eps):
    """residual += x (in place, bf16); returns rms_norm(residual)."""
    _req(x, _BF16, "x"); _req(residual, _BF16, "residual")
    M, N = x.shape
    y = torch.empty_like(x)
    check(lib.teeny_add_rms_norm_bf16(_ptr(x), _ptr(residual), _ptr(y), _ptr(weight), M, N, float(eps), _stream()),
          "add_rms_norm")
    return y


def silu_mul(gate_up):
    _req(gate_up, _BF16, "gate_up")
    T, two_i = gate_up.shape
    out = torch.empty(T, two_i // 2, dtype=_BF16, device=gate_up.device)
    check(lib.teeny_silu_mul_bf16(_ptr(gate_up), gate_up.stride(0), _ptr(out), T, two_i // 2, _stream()), "silu_mul")
    return out


def interleave_gate_up(gate_w, up_w):
    """Fused SwiGLU weight layout: blocks of 64 gate rows followed by the 64 up rows of the same channels."""
    I, K = gate_w.shape
    if I % 64:
        raise ValueError("intermediate size must be a multiple of 64")
    return torch.stack([gate_w.view(I // 64, 64, K), up_w.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def linear_swiglu(x, w_interleaved, out=None):
    """silu(x @ Wg^T) * (x @ Wu^T) with Wg / Wu interleaved by ``interleave_gate_up``; x [M,K] -> [M, N/2]."""
    _req(x, _BF16, "x"); _req(w_interleaved, _BF16, "w")
    M, K = x.shape
    N = w_interleaved.shape[0]
    out = torch.empty(M, N // 2, dtype=_BF16, device=x.device) if out is None else out
    check(lib.teeny_linear_swiglu_bf16(_ptr(x), x.stride(0), _ptr(w_interleaved), w_interleaved.stride(0), _ptr(out),
                                       out.stride(0), M, N, K, _stream()), "linear_swiglu")
    return out


SCALE_KINDS = {"tensor": 0, "channel": 1, "group": 2}


def _as_bytes(w):
    if w.dtype == torch.uint8:
        return w
    if w.dtype == torch.float8_e4m3fn:
        return w.view(torch.uint8)
    raise ValueError(f"FP8 weight must be uint8 or float8_e4m3fn, got {w.dtype}")


def linear_w8a16(x, w_fp8, w_scale, strategy="channel", group_size=0, bias=None, out=None, scratch=None, swiglu=False):
    """x [M, K] bf16 times an FP8 (E4M3) weight [N, K] with float32 scales (``strategy`` "tensor" | "channel" | "group",
    the reference quantiser's names); swiglu: rows interleaved by ``interleave_gate_up`` (scales too), out [M, N/2].
    M > 128 needs ``scratch`` of ``lib.teeny_linear_w8a16_scratch_bytes`` bytes (allocated here when not given)."""
    _req(x, _BF16, "x"); _req(w_scale, _F32, "w_scale")
    w = _req(_as_bytes(w_fp8), torch.uint8, "w_fp8")
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty(M, N // 2 if swiglu else N, dtype=_BF16, device=x.device) if out is None else out
    need = lib.teeny_linear_w8a16_scratch_bytes(M, N, K)
    if need and scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.teeny_linear_w8a16_forward(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(w_scale), SCALE_KINDS[strategy],
                                         group_size, _ptr(bias), _ptr(out), out.stride(0), M, N, K, int(swiglu),
                                         _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()),
          "linear_w8a16")
    return out


def split_fp8(x, out=None, scale=None):
    """x [M, K] bf16 -> (bytes [2 * M, K]: the E4M3 hi terms, then the lo terms times 16; x_scale [M] = 1 / s), with
    x * s = hi + lo exactly wherever both terms are normal E4M3 numbers."""
    _req(x, _BF16, "x")
    M, K = x.shape
    out = torch.empty(2 * M, (K + 15) // 16 * 16, dtype=torch.uint8, device=x.device)[:, :K] if out is None else out
    scale = torch.empty(M, dtype=_F32, device=x.device) if scale is None else scale
    check(lib.teeny_split_fp8_e4m3(_ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(scale), M, K, _stream()), "split_fp8")
    return out, scale


def linear_w8a8x2(x8, x_scale, w_fp8, w_scale, strategy="channel", bias=None, out=None, swiglu=False):
    """FP8 weights times two-term FP8 activations (``split_fp8``): [M, N] bf16 (or [M, N / 2] with swiglu), M <= 128."""
    _req(x8, torch.uint8, "x8"); _req(x_scale, _F32, "x_scale"); _req(w_scale, _F32, "w_scale")
    w = _req(_as_bytes(w_fp8), torch.uint8, "w_fp8")
    M, K = x8.shape[0] // 2, x8.shape[1]
    N = w.shape[0]
    out = torch.empty(M, N // 2 if swiglu else N, dtype=_BF16, device=x8.device) if out is None else out
    check(lib.teeny_linear_w8a8x2_forward(_ptr(x8), x8.stride(0), _ptr(x_scale), _ptr(w), w.stride(0), _ptr(w_scale),
                                          SCALE_KINDS[strategy], _ptr(bias), _ptr(out), out.stride(0), M, N, K, int(swiglu),
                                          _stream()), "linear_w8a8x2")
    return out


def dequant_fp8(w_fp8, w_scale, strategy="channel", group_size=0, out=None):
    """bf16(decode(byte) * scale) of an FP8 (E4M3) tensor [N, K]."""
    w = _req(_as_bytes(w_fp8), torch.uint8, "w_fp8"); _req(w_scale, _F32, "w_scale")
    N, K = w.shape
    out = torch.empty(N, K, dtype=_BF16, device=w.device) if out is None else out
    check(lib.teeny_dequant_fp8_e4m3_bf16(_ptr(w), w.stride(0), _ptr(w_scale), SCALE_KINDS[strategy], group_size, _ptr(out),
                                          out.stride(0), N, K, _stream()), "dequant_fp8")
    return out


def dequant_int(q, bits, w_scale, zero_point, shape, strategy="channel", group_size=0, out=None):
    """bf16((q - zero_point) * scale) of an integer-quantised matrix of logical ``shape`` [N, K]: ``q`` int8 [N, K]
    (bits 8) or the packed uint8 vector of the 4-bit scheme (bits 4); ``zero_point`` int32 per group or None."""
    N, K = shape
    q = q.contiguous()
    _req(q, name="q"); _req(w_scale, _F32, "w_scale")
    if zero_point is not None:
        _req(zero_point, torch.int32, "zero_point")
    if q.numel() != (N * K if bits == 8 else (N * K + 1) // 2):
        raise ValueError("quantised tensor does not have the size its logical shape implies")
    out = torch.empty(N, K, dtype=_BF16, device=q.device) if out is None else out
    check(lib.teeny_dequant_int_bf16(_ptr(q), bits, _ptr(w_scale), _ptr(zero_point), SCALE_KINDS[strategy], group_size,
                                     _ptr(out), out.stride(0), N, K, _stream()), "dequant_int")
    return out


def fp8_count_nan(w_fp8):
    w = _req(_as_bytes(w_fp8), torch.uint8, "w_fp8").contiguous()
    count = torch.zeros(1, dtype=torch.int32, device=w.device)
    check(lib.teeny_fp8_e4m3_count_nan(_ptr(w), w.numel(), _ptr(count), _stream()), "fp8_count_nan")
    return int(count.item())


def rope_table(inv_freq, max_pos):
    _req(inv_freq, _F32, "inv_freq")
    D = inv_freq.numel() * 2
    cos = torch.empty(max_pos, D, dtype=_BF16, device=inv_freq.device)
    sin = torch.empty_like(cos)
    check(lib.teeny_rope_table_bf16(_ptr(inv_freq), _ptr(cos), _ptr(sin), max_pos, D, _stream()), "rope_table")
    return cos, sin


def qk_norm_rope_kv(qkv, q_w, k_w, cos, sin, k_cache, v_cache, S, Hq, Hkv, pos0, eps):
    """In-place per-head norm + RoPE on the q part of qkv [T, (Hq+2Hkv)*D]; k, v appended to the caches."""
    _req(qkv, _BF16, "qkv")
    T = qkv.shape[0]
    D = k_cache.shape[-1]
    dev_pos = pos0 if torch.is_tensor(pos0) else None
    check(lib.teeny_qk_norm_rope_kv_bf16(_ptr(qkv), qkv.stride(0), _ptr(q_w), _ptr(k_w), _ptr(cos), _ptr(sin),
                                         _ptr(k_cache), _ptr(v_cache), T, S, Hq, Hkv, D, k_cache.shape[2],
                                         0 if dev_pos is not None else int(pos0), _ptr(dev_pos), float(eps),
                                         _stream()), "qk_norm_rope_kv")


def embedding(ids, table):
    _req(ids, torch.int32, "ids"); _req(table, _BF16, "table")
    out = torch.empty(ids.numel(), table.shape[1], dtype=_BF16, device=table.device)
    check(lib.teeny_embedding_bf16(_ptr(ids), _ptr(table), _ptr(out), ids.numel(), table.shape[1], table.shape[0],
                                   _stream()), "embedding")
    return out


def argmax(logits, idx_offset=0):
    """Row argmax of bf16 logits [rows, cols] -> (values f32 [rows], indices int32 [rows])."""
    _req(logits, _BF16, "logits")
    rows, cols = logits.shape
    val = torch.empty(rows, dtype=_F32, device=logits.device)
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib.teeny_argmax_bf16(_ptr(logits), logits.stride(0), _ptr(val), _ptr(idx), rows, cols, idx_offset,
                                _stream()), "argmax")
    return val, idx


def argmax_combine(vals, idx):
    parts, rows = vals.shape
    out = torch.empty(rows, dtype=torch.int32, device=vals.device)
    check(lib.teeny_argmax_combine(_ptr(vals), _ptr(idx), _ptr(out), parts, rows, _stream()), "argmax_combine")
    return out


def sample_top_k_top_p(logits, temperature, top_k, top_p, u, want_prob=False):
    """Temperature / top-k / top-p sampling of one token per row of bf16 logits [rows, cols]; ``u`` f32 [rows] in
    [0, 1) supplies the randomness (the call itself is deterministic).  Returns indices int32 [rows] (and the sampled
    tokens' probabilities inside the nucleus when asked)."""
    _req(logits, _BF16, "logits"); _req(u, _F32, "u")
    rows, cols = logits.shape
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    prob = torch.empty(rows, dtype=_F32, device=logits.device) if want_prob else None
    check(lib.teeny_sample_top_k_top_p_bf16(_ptr(logits), logits.stride(0), rows, cols, float(temperature), int(top_k),
                                            float(top_p), _ptr(u), _ptr(idx), _ptr(prob), _stream()),
          "sample_top_k_top_p")
    return (idx, prob) if want_prob else idx
