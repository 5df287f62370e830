"""Host side of the FP8 path on the CPU: the quantised-checkpoint layout of the reference's quantiser
(utilities/teeny-quant/src/format.rs), scale bookkeeping under fusion and tensor-parallel sharding."""
import json

import numpy as np
import pytest
import torch

from teenygrad_b200 import quant
from teenygrad_b200 import safetensors as st


def _meta(**weights):
    base = dict(num_bits=8, type="float", symmetric=True, fp8_variant="e4m3")
    base.update(weights)
    return {"quantization_config": json.dumps({"quant_method": "compressed-tensors", "format": "float-quantized",
                                               "config_groups": {"group_0": {"weights": base, "targets": ["*"]}},
                                               "ignore": ["model.norm.weight"]})}


def test_parse_quantization_config_accepts_the_three_strategies():
    s, ign = quant.parse_quantization_config(_meta(strategy="tensor"))
    assert (s.strategy, s.group_size) == ("tensor", 0) and ign == ["model.norm.weight"]
    assert quant.parse_quantization_config(_meta(strategy="channel", axis=0))[0].strategy == "channel"
    s, _ = quant.parse_quantization_config(_meta(strategy="group", axis=1, group_size=128))
    assert (s.strategy, s.group_size) == ("group", 128)


@pytest.mark.parametrize("bad", [
    dict(strategy="channel", axis=1),                 # scales along the input axis
    dict(strategy="group", axis=1, group_size=32),    # not a multiple of the kernel's 64-wide k-block
    dict(strategy="group", axis=0, group_size=64),
    dict(strategy="tensor", fp8_variant="e5m2"),
    dict(strategy="tensor", type="int"),
    dict(strategy="block"),
])
def test_parse_quantization_config_refuses_what_the_kernels_do_not_take(bad):
    with pytest.raises(ValueError):
        quant.parse_quantization_config(_meta(**bad))
    with pytest.raises(ValueError):
        quant.parse_quantization_config({})


def test_scales_follow_rows_columns_fusion_and_interleave():
    from oracle import quant as oq
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((256, 512)) * 0.1).astype(np.float32)
    for strategy, kw, scheme in (("tensor", {}, quant.Fp8Scheme("tensor")),
                                 ("channel", {"axis": 0}, quant.Fp8Scheme("channel")),
                                 ("group", {"axis": 1, "group_size": 128}, quant.Fp8Scheme("group", 128))):
        q, s = oq.quantize_fp8(w, strategy, **kw)
        full = torch.from_numpy(oq.dequantize_fp8(q, s, strategy, **kw))
        fw = quant.Fp8Weight.from_tensors(torch.from_numpy(q), torch.from_numpy(s), scheme)
        assert torch.equal(fw.dequantize(), full)
        assert torch.equal(fw.rows(64, 192).dequantize(), full[64:192])
        assert torch.equal(fw.cols(128, 384).dequantize(), full[:, 128:384])
        fused = quant.Fp8Weight.cat_rows([fw.rows(0, 128), fw.rows(128, 256)])
        assert torch.equal(fused.dequantize(), full)
        il = quant.Fp8Weight.interleave(fw.rows(0, 128), fw.rows(128, 256)).dequantize()
        assert torch.equal(il[:64], full[:64]) and torch.equal(il[64:128], full[128:192])
        assert torch.equal(il[128:192], full[64:128]) and torch.equal(il[192:], full[192:])
    with pytest.raises(ValueError):
        fw.cols(64, 256)  # a column shard that cuts a scale group


def test_quantized_checkpoint_round_trips_through_a_file(tmp_path):
    """quantize_state_dict writes the layout parse_quantization_config / Fp8Weight.from_tensors read back, and the
    safetensors package (what the reference's crate implements) sees the same FP8 bytes."""
    g = torch.Generator().manual_seed(1)
    sd = {"model.layers.0.mlp.down_proj.weight": torch.randn(64, 128, generator=g).bfloat16(),
          "model.norm.weight": torch.ones(64).bfloat16()}
    tensors, meta = quant.quantize_state_dict(sd, "group", 64)
    st.save_file(tensors, tmp_path / "q.safetensors", metadata=meta)
    ck = st.SafeTensors(tmp_path / "q.safetensors")
    scheme, ignore = quant.parse_quantization_config(ck.metadata)
    assert ignore == ["model.norm.weight"] and ck["model.norm.weight"].dtype == torch.bfloat16
    name = "model.layers.0.mlp.down_proj.weight"
    assert ck[name].dtype == torch.float8_e4m3fn and ck[name + "_scale"].shape == (64 * 2,)
    w = quant.Fp8Weight.from_tensors(ck[name], ck[name + "_scale"], scheme)
    err = (w.dequantize() - sd[name].float()).abs().max() / sd[name].float().abs().max()
    assert err < 2.0 ** -4
    safetensors_torch = pytest.importorskip("safetensors.torch")
    theirs = safetensors_torch.load_file(str(tmp_path / "q.safetensors"))
    assert torch.equal(theirs[name].view(torch.uint8), ck[name].view(torch.uint8))


def test_torch_encoder_equals_the_reference_encoder_on_normal_values():
    """quant.quantize_fp8 (PyTorch's cast) and the reference's encoder (oracle) agree wherever no quotient falls under
    E4M3's smallest normal."""
    from oracle import quant as oq
    g = torch.Generator().manual_seed(2)
    w = torch.randn(32, 256, generator=g) * 0.05
    w = torch.where(w.abs() < w.abs().amax(dim=1, keepdim=True) * 2.0 ** -5, torch.zeros_like(w), w)
    ours = quant.quantize_fp8(w, "channel")
    q, s = oq.quantize_fp8(w.numpy(), "channel", axis=0)
    assert np.array_equal(ours.scale.numpy(), s) and np.array_equal(ours.q.numpy(), q)


def test_parse_quantization_config_integer_formats():
    meta = {"quantization_config": json.dumps({
        "quant_method": "compressed-tensors", "format": "pack-quantized",
        "config_groups": {"group_0": {"weights": dict(num_bits=4, type="int", symmetric=False, strategy="group", axis=1,
                                                      group_size=64), "targets": ["*"]}},
        "teenygrad_packed_int4": {"a.weight": {"logical_shape": [4, 8], "elements": 32}}})}
    s, _ = quant.parse_quantization_config(meta)
    assert isinstance(s, quant.IntScheme) and (s.bits, s.symmetric, s.strategy, s.group_size) == (4, False, "group", 64)
    assert s.packed_shapes == {"a.weight": (4, 8)}
    meta8 = {"quantization_config": json.dumps({
        "quant_method": "compressed-tensors", "format": "int-quantized",
        "config_groups": {"group_0": {"weights": dict(num_bits=8, type="int", symmetric=True, strategy="channel", axis=0),
                                      "targets": ["*"]}}})}
    s, _ = quant.parse_quantization_config(meta8)
    assert (s.bits, s.symmetric, s.strategy) == (8, True, "channel")
    bad = json.loads(meta8["quantization_config"])
    bad["config_groups"]["group_0"]["weights"]["num_bits"] = 4  # int-quantized is the 8-bit format
    with pytest.raises(ValueError):
        quant.parse_quantization_config({"quantization_config": json.dumps(bad)})
