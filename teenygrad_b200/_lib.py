"""ctypes binding of libteeny_b200.so.  Signatures follow include/teeny_b200.h one to one."""
import ctypes as C
import os

from .build import library_path

_path = library_path()
if not os.path.exists(_path):
    raise ImportError(
        f"{_path} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` (or `make -C "
        "teenygrad_b200/csrc`).  This backend has no CPU or PyTorch fallback.")
lib = C.CDLL(_path)

vp, i32, f32, i64, sz = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_size_t


class AttnShape(C.Structure):
    """teeny_attn_shape"""
    _fields_ = [(n, i32) for n in ("B", "Hq", "Hkv", "Sq", "Skv", "D")] + \
               [(n, i64) for n in ("q_sb", "q_sh", "q_ss", "k_sb", "k_sh", "k_ss",
                                   "v_sb", "v_sh", "v_ss", "o_sb", "o_sh", "o_ss")] + \
               [("scale", f32), ("causal", i32)]


SIGNATURES = {
    "teeny_version": (i32, []),
    "teeny_status_string": (C.c_char_p, [i32]),
    "teeny_device_error": (i32, [i32]),
    "teeny_launch_count": (C.c_ulonglong, [i32]),
    "matmul_forward_entry_point_f32": (i32, [vp, vp, vp, i32, i32, i32, vp, sz, vp]),
    "matmul_forward_entry_point_bf16": (i32, [vp, vp, vp, i32, i32, i32, vp, sz, vp]),
    "linear_forward_entry_point_f32": (i32, [vp, vp, vp, vp] + [i32] * 9 + [vp, sz, vp]),
    "linear_forward_entry_point_bf16": (i32, [vp, vp, vp, vp] + [i32] * 9 + [vp, sz, vp]),
    "teeny_gemm_scratch_bytes": (sz, [i32, i32, i32]),
    "teeny_matmul_f32_scratch_bytes": (sz, [i32, i32, i32]),
    "flash_attention2_forward_entry_point_f32": (i32, [vp, vp, vp, vp, vp, i32, i32, f32, f32, i32, i32, vp]),
    "flash_attention2_forward_entry_point_bf16": (i32, [vp, vp, vp, vp, vp, i32, i32, f32, f32, i32, i32, vp]),
    "teeny_flash_attn_fwd_bf16": (i32, [vp, vp, vp, vp, vp, C.POINTER(AttnShape), vp]),
    "teeny_flash_attn_decode_bf16": (i32, [vp, vp, vp, vp, C.POINTER(AttnShape), i32, vp, vp, sz, vp]),
    "teeny_attn_decode_scratch_bytes": (sz, [i32, i32, i32, i32]),
    "teeny_flash_attn_decode_bf16_static": (i32, [vp, vp, vp, vp, C.POINTER(AttnShape), i32, vp, vp]),
    "teeny_attn_decode_static_limit": (sz, []),
    "rms_norm_forward_entry_point_f32": (i32, [vp, vp, vp, vp, i32, i32, f32, vp]),
    "rms_norm_forward_entry_point_bf16": (i32, [vp, vp, vp, vp, i32, i32, f32, vp]),
    "silu_forward_entry_point_f32": (i32, [vp, vp, i32, vp]),
    "silu_forward_entry_point_bf16": (i32, [vp, vp, i32, vp]),
    "elemwise_mul_forward_entry_point_f32": (i32, [vp, vp, vp, i32, vp]),
    "elemwise_mul_forward_entry_point_bf16": (i32, [vp, vp, vp, i32, vp]),
    "elemwise_add_forward_entry_point_f32": (i32, [vp, vp, vp, i32, vp]),
    "elemwise_add_forward_entry_point_bf16": (i32, [vp, vp, vp, i32, vp]),
    "softmax_forward_entry_point_f32": (i32, [vp, vp, i32, i32, vp]),
    "softmax_forward_entry_point_bf16": (i32, [vp, vp, i32, i32, vp]),
    "teeny_add_rms_norm_bf16": (i32, [vp, vp, vp, vp, i32, i32, f32, vp]),
    "teeny_silu_mul_bf16": (i32, [vp, i64, vp, i32, i32, vp]),
    "teeny_linear_swiglu_bf16": (i32, [vp, i64, vp, i64, vp, i64, i32, i32, i32, vp]),
    "teeny_linear_w8a16_forward": (i32, [vp, i64, vp, i64, vp, i32, i32, vp, vp, i64, i32, i32, i32, i32, vp, sz, vp]),
    "teeny_linear_w8a16_scratch_bytes": (sz, [i32, i32, i32]),
    "teeny_split_fp8_e4m3": (i32, [vp, i64, vp, i64, vp, i32, i32, vp]),
    "teeny_linear_w8a8x2_forward": (i32, [vp, i64, vp, vp, i64, vp, i32, vp, vp, i64, i32, i32, i32, i32, vp]),
    "teeny_dequant_fp8_e4m3_bf16": (i32, [vp, i64, vp, i32, i32, vp, i64, i32, i32, vp]),
    "teeny_fp8_e4m3_count_nan": (i32, [vp, sz, vp, vp]),
    "teeny_dequant_int_bf16": (i32, [vp, i32, vp, vp, i32, i32, vp, i64, i32, i32, vp]),
    "teeny_rope_table_bf16": (i32, [vp, vp, vp, i32, i32, vp]),
    "teeny_qk_norm_rope_kv_bf16": (i32, [vp, i64, vp, vp, vp, vp, vp, vp] + [i32] * 7 + [vp, f32, vp]),
    "teeny_embedding_bf16": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "teeny_argmax_bf16": (i32, [vp, i64, vp, vp, i32, i32, i32, vp]),
    "teeny_argmax_combine": (i32, [vp, vp, vp, i32, i32, vp]),
    "teeny_sample_top_k_top_p_bf16": (i32, [vp, i64, i32, i32, f32, i32, f32, vp, vp, vp, vp]),
    "teeny_sample_candidates_bf16": (i32, [vp, i64, i32, i32, i32, i32, vp, vp]),
    "teeny_sample_merge": (i32, [vp, i32, sz, i32, f32, i32, f32, vp, vp, vp, vp]),
}


def bind(signatures):
    for name, (res, args) in signatures.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype, fn.argtypes = res, args


bind(SIGNATURES)


class TeenyError(RuntimeError):
    pass


def check(status, what):
    if status != 0:
        msg = lib.teeny_status_string(status).decode()
        raise TeenyError(f"{what}: status {status} ({msg})")
