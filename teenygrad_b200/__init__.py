"""teenygrad_b200: sm_100a (B200) backend for teenygrad's GEMM / flash-attention / Qwen3-forward path.

The compute lives in ``libteeny_b200.so`` (hand-written CUDA behind the C ABI declared in
``include/teeny_b200.h``).  This package is the host side: a ctypes binding (``_lib``), thin operator
wrappers over torch device tensors (``ops``), tensor-parallel sharding (``tp``), a safetensors reader
(``safetensors``) and the Qwen3 runner (``qwen3``).  There is no CPU fallback: importing ``_lib`` fails when the library has not
been built, and every operator raises when the C ABI returns a non-zero status.
"""
from .build import build, library_path  # noqa: F401

__all__ = ["build", "library_path"]
