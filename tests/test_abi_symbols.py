"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments before touching a device (no kernel runs here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as g
    g.build()
    from teenygrad_b200 import _lib
    return _lib


def _declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b([a-z][a-z0-9_]+)\s*\([^;{]*\)\s*;", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_functions()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib.lib, name), f"{name} declared in include/ but not exported"
    bound = set(lib.SIGNATURES)
    try:
        from teenygrad_b200 import qwen3
        bound |= set(getattr(qwen3, "SIGNATURES", {}))
    except ImportError:
        pass
    assert set(declared) <= bound, sorted(set(declared) - bound)


def test_status_strings_and_argument_checks(lib):
    assert lib.lib.teeny_version() >= 100
    assert b"alignment" in lib.lib.teeny_status_string(-2)
    # null pointers / bad sizes are rejected on the host, before any CUDA call
    assert lib.lib.linear_forward_entry_point_bf16(None, None, None, None, 4, 4, 8, 8, 1, 8, 1, 4, 1, None, 0, None) == -1
    assert lib.lib.silu_forward_entry_point_f32(None, None, 16, None) == -1
    assert lib.lib.teeny_flash_attn_fwd_bf16(None, None, None, None, None, None, None) == -1
    assert lib.lib.teeny_gemm_scratch_bytes(4096, 4096, 4096) == 0
