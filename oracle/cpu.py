"""CPU oracle kernels (test infrastructure only; the product never imports this module).

f32 entry points call the C restatement in ``teeny_oracle.c`` through ctypes; each C function cites
the reference source it follows.  The bf16 variants have no counterpart in the reference (its
kernels are f32/f64 only, ``macros/teeny-macros/src/macros/kernel.rs:81-98``); they apply the same
formulas with PyTorch CPU on bf16 inputs up-cast to f32, f32 accumulation, one rounding to bf16 at
the output -- the semantics of ``F.linear`` / SDPA that the reference's fixture generator
(``kernels/teeny-kernels/tests/fixtures/generate.py``) and its Qwen3 trace are built on.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libteeny_oracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)


def build():
    """Compile ``teeny_oracle.c`` (gcc) if the shared object is missing or stale."""
    src = os.path.join(_HERE, "teeny_oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def matmul_f32(a, b):
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float32)
    lib().oracle_matmul_f32(_p(a), _p(b), _p(c), M, N, K)
    return c


def linear_f32(x, w, bias=None):
    x, w, bias = _c(x), _c(w), _c(bias)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), np.float32)
    lib().oracle_linear_f32(_p(x), _p(w), _p(bias), _p(y), M, N, K)
    return y


def attention_f32(q, k, v, scale, causal=False):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] -> (o [B,Hq,Sq,D], lse [B,Hq,Sq])."""
    q, k, v = _c(q), _c(k), _c(v)
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    o = np.empty_like(q)
    lse = np.empty((B, Hq, Sq), np.float32)
    lib().oracle_attention_f32(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Hq, Hkv, Sq, Skv, D,
                               ctypes.c_float(scale), int(bool(causal)))
    return o, lse


def rms_norm_f32(x, weight, eps):
    x, weight = _c(x), _c(weight)
    M, N = x.shape
    y = np.empty_like(x)
    rrms = np.empty((M,), np.float32)
    lib().oracle_rms_norm_f32(_p(x), _p(y), _p(weight), _p(rrms), M, N, ctypes.c_float(eps))
    return y, rrms


def _unary(fn, x):
    x = _c(x)
    y = np.empty_like(x)
    fn(_p(x), _p(y), x.size)
    return y


def _binary(fn, a, b):
    a, b = _c(a), _c(b)
    out = np.empty_like(a)
    fn(_p(a), _p(b), _p(out), a.size)
    return out


def silu_f32(x):
    return _unary(lib().oracle_silu_f32, x)


def mul_f32(a, b):
    return _binary(lib().oracle_mul_f32, a, b)


def add_f32(a, b):
    return _binary(lib().oracle_add_f32, a, b)


def softmax_f32(x):
    x = _c(x)
    y = np.empty_like(x)
    lib().oracle_softmax_f32(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


# ---------------------------------------------------------------------------------------------
# bf16 variants (PyTorch CPU; f32 accumulate, round once to bf16)
# ---------------------------------------------------------------------------------------------

def linear_bf16(x, w, bias=None):
    """x [M,K] bf16, w [N,K] bf16 -> bf16 [M,N]; f32 accumulation (up-cast then F.linear)."""
    y = torch.nn.functional.linear(x.float(), w.float(), None if bias is None else bias.float())
    return y.to(torch.bfloat16)


def matmul_bf16(a, b):
    """a [M,K] bf16, b [K,N] bf16 (row-major, the matmul_forward layout) -> bf16 [M,N]."""
    return (a.float() @ b.float()).to(torch.bfloat16)


def attention_bf16(q, k, v, scale, causal=True):
    """bf16 q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D]; f32 softmax; returns (o bf16, lse f32).

    Scores, softmax and PV in f32 from the bf16 inputs (probabilities are NOT re-rounded to bf16):
    this is the mathematical target the 2e-2 bound is measured against."""
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(Sq).unsqueeze(1)
        j = torch.arange(Skv).unsqueeze(0)
        s = s.masked_fill(j > i + (Skv - Sq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.to(torch.bfloat16), lse


def rms_norm_bf16(x, weight, eps):
    """HF/Qwen3 rounding points: statistics in f32, down-cast to bf16, THEN multiply by the bf16 weight."""
    h = x.float()
    var = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(var + eps)
    return weight * h.to(torch.bfloat16)


def silu_mul_bf16(gate, up):
    """bf16 silu(gate) (computed in f32, rounded to bf16) times up, rounded to bf16."""
    return torch.nn.functional.silu(gate) * up
