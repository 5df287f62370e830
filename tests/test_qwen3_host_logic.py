"""Host-side checks of the Qwen3 runner wrapper that need no GPU."""
import pytest


def test_generation_must_fit_the_cache_and_the_history():
    from teenygrad_b200.qwen3 import check_generation_fits
    check_generation_fits(prompt_len=2048, max_new_tokens=256, max_len=2304, history_capacity=256)
    check_generation_fits(prompt_len=8, max_new_tokens=3, max_len=10, history_capacity=8)
    with pytest.raises(ValueError, match="cache rows"):
        check_generation_fits(prompt_len=8, max_new_tokens=4, max_len=10, history_capacity=8)
    with pytest.raises(ValueError, match="history"):
        check_generation_fits(prompt_len=8, max_new_tokens=9, max_len=100, history_capacity=8)
