"""The no-allocation decode-attention entry point (teeny_flash_attn_decode_bf16_static) against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other
test.  The static entry point is for hosts that cannot give the library scratch memory once serving has started
(all of HBM already belongs to their own pool; a cudaMalloc would synchronise the device in the middle of the decode
loop), so the test calls it the way such a host would: through the C ABI, with only inputs and outputs, twice in a
row -- the second call finds the built-in array holding the first call's partials and must still be right.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu



def _shape(lib_mod, q, k, v, o, scale):
    s = lib_mod.AttnShape()
    s.B, s.Hq, s.Hkv, s.Sq, s.Skv, s.D = q.shape[0], q.shape[1], k.shape[1], 1, k.shape[2], q.shape[3]
    s.q_sb, s.q_sh, s.q_ss = q.stride(0), q.stride(1), q.stride(2)
    s.k_sb, s.k_sh, s.k_ss = k.stride(0), k.stride(1), k.stride(2)
    s.v_sb, s.v_sh, s.v_ss = v.stride(0), v.stride(1), v.stride(2)
    s.o_sb, s.o_sh, s.o_ss = o.stride(0), o.stride(1), o.stride(2)
    s.scale, s.causal = scale, 0
    return s


def test_static_entry_point_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from teenygrad_b200 import _lib
    lib = _lib.lib
    vp = C.c_void_p
    stream = vp(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(12)
    for call, (B, Hq, Hkv, cap, L) in enumerate([(4, 16, 4, 1536, 1100), (2, 8, 2, 640, 640)]):
        q = torch.randn(B, Hq, 1, 128, generator=g).bfloat16().cuda()
        k = torch.randn(B, Hkv, cap, 128, generator=g).bfloat16().cuda()
        v = torch.randn(B, Hkv, cap, 128, generator=g).bfloat16().cuda()
        want, got = torch.empty_like(q), torch.empty_like(q)
        s = _shape(_lib, q, k, v, want, 128 ** -0.5)
        need = lib.teeny_attn_decode_scratch_bytes(B, Hq, 128, cap)
        assert need <= lib.teeny_attn_decode_static_limit()
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        st = lib.teeny_flash_attn_decode_bf16(vp(q.data_ptr()), vp(k.data_ptr()), vp(v.data_ptr()), vp(want.data_ptr()),
                                              C.byref(s), L, None, vp(scratch.data_ptr()), need, stream)
        assert st == 0, lib.teeny_status_string(st)
        st = lib.teeny_flash_attn_decode_bf16_static(vp(q.data_ptr()), vp(k.data_ptr()), vp(v.data_ptr()),
                                                     vp(got.data_ptr()), C.byref(s), L, None, stream)
        assert st == 0, lib.teeny_status_string(st)
        torch.cuda.synchronize()
        # the two entry points run the same kernels on the same split, only the partials live elsewhere: bit-identical
        assert torch.equal(got, want), f"call {call}: static entry point differs from the regular one by " \
            f"{float((got.float() - want.float()).abs().max())}"
    assert lib.teeny_device_error(1) == 0


def test_static_entry_point_rejects_shapes_beyond_its_built_in_scratch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from teenygrad_b200 import _lib
    lib = _lib.lib
    B, Hq, Hkv, cap = 64, 64, 8, 16384  # 64*64*32 chunks*130*4 B = 68 MB of partials: above the 8 MiB built in
    assert lib.teeny_attn_decode_scratch_bytes(B, Hq, 128, cap) > lib.teeny_attn_decode_static_limit()
    q = torch.zeros(B, Hq, 1, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, Hkv, 8, 128, dtype=torch.bfloat16, device="cuda")  # never read: the call is refused first
    s = _shape(_lib, q, k, k, q, 1.0)
    s.Skv = cap
    vp = C.c_void_p
    st = lib.teeny_flash_attn_decode_bf16_static(vp(q.data_ptr()), vp(k.data_ptr()), vp(k.data_ptr()), vp(q.data_ptr()),
                                                 C.byref(s), 8, None, vp(torch.cuda.current_stream().cuda_stream))
    assert st == -7
    assert b"no-allocation" in lib.teeny_status_string(st)
