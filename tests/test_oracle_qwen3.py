"""The plain-PyTorch Qwen3 restatement must reproduce HF transformers' Qwen3ForCausalLM (the code the
reference's Qwen3 script actually executes, support/teeny-torch/python/tests/test_qwen3.py:24-41) on the
same seeded random weights: identical greedy ids and logits equal to bf16 rounding."""
import pytest
import torch

from oracle import qwen3 as oq


@pytest.mark.parametrize("tied", [True, False])
def test_restatement_matches_transformers(tied):
    pytest.importorskip("transformers")
    cfg = oq.OracleQwen3Config(2, 256, 4, 2, 128, 512, 1000, tied=tied)
    sd = oq.make_weights(cfg, 3)
    ids = torch.randint(0, cfg.vocab, (2, 17), generator=torch.Generator().manual_seed(0))
    mine, logits = oq.OracleQwen3(cfg, sd).generate(ids, 6, return_logits=True)
    hf = oq.hf_model(cfg, sd)
    out = hf.generate(ids, max_new_tokens=6, do_sample=False, return_dict_in_generate=True, output_logits=True)
    assert torch.equal(out.sequences[:, 17:], mine)
    hl = torch.stack(out.logits, 1).float()
    assert (hl - logits.float()).abs().max() <= 2e-2 * logits.float().abs().max()


def test_rope_tables_shape_and_values():
    cfg = oq.OracleQwen3Config(1, 256, 2, 1, 128, 512, 100)
    cos, sin = oq.rope_tables(cfg, torch.arange(4))
    assert cos.shape == (4, 128) and cos.dtype == torch.bfloat16
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)
    assert torch.equal(cos[:, :64], cos[:, 64:])
