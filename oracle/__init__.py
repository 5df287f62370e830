"""CPU oracle for the hot path -- TEST INFRASTRUCTURE, never imported by the product package.

``oracle.cpu``   : f32 kernels restated in C (``teeny_oracle.c``) plus bf16 variants in PyTorch CPU.
``oracle.qwen3`` : the Qwen3 decoder forward restated op by op in plain PyTorch.
"""
