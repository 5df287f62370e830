"""safetensors reader / writer and the Hugging Face Qwen3 checkpoint layout (host logic, no GPU)."""
import json
import struct

import pytest
import torch

from oracle import qwen3 as oq
from teenygrad_b200 import safetensors as st
from teenygrad_b200 import tp
from teenygrad_b200.qwen3 import Qwen3Config


def _tensors():
    g = torch.Generator().manual_seed(0)
    return {
        "a.bf16": torch.randn(7, 33, generator=g).bfloat16(),
        "b.f32": torch.randn(5, generator=g),
        "c.f16": torch.randn(2, 3, 4, generator=g).half(),
        "d.i64": torch.arange(6).view(2, 3),
        "e.scalar": torch.tensor(3.5),
        "f.empty": torch.empty(0, 4),
        "g.bool": torch.tensor([True, False, True]),
    }


def test_round_trip_is_bit_exact(tmp_path):
    tensors = _tensors()
    path = tmp_path / "x.safetensors"
    st.save_file(tensors, path, {"format": "pt"})
    back = st.SafeTensors(path)
    assert sorted(back) == sorted(tensors) and back.metadata == {"format": "pt"}
    for name, t in tensors.items():
        got = back[name]
        assert got.dtype == t.dtype and got.shape == t.shape
        if t.numel():  # compare the bytes (NaN-safe, dtype-agnostic)
            assert torch.equal(got.reshape(-1).view(torch.uint8), t.reshape(-1).view(torch.uint8))


def test_file_layout_matches_the_format(tmp_path):
    path = tmp_path / "y.safetensors"
    st.save_file({"w": torch.arange(4, dtype=torch.float32)}, path)
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    assert header == {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}
    assert raw[8 + n:] == torch.arange(4, dtype=torch.float32).numpy().tobytes()


def test_corrupt_headers_are_rejected(tmp_path):
    path = tmp_path / "z.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        st.SafeTensors(path)
    js = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(js)) + js + b"\0" * 16)
    with pytest.raises(ValueError):
        st.SafeTensors(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError):
        st.SafeTensors(path)


def test_sharded_qwen3_checkpoint_gives_the_same_rank_shards(tmp_path):
    ocfg = oq.OracleQwen3Config(2, 256, 4, 2, 128, 512, 1024, tied=False)
    sd = oq.make_weights(ocfg, 11)
    files = st.save_sharded(sd, tmp_path / "ckpt", max_shard_bytes=600_000)
    assert len(files) > 1
    ckpt = st.SafeTensors(tmp_path / "ckpt")
    assert sorted(ckpt) == sorted(sd)
    cfg = Qwen3Config(2, 256, 4, 2, 128, 512, 1024, tied=False)
    for world in (1, 2):
        for rank in range(world):
            for layer in range(cfg.num_layers):
                want = tp.shard_layer(sd, cfg, layer, rank, world)
                got = tp.shard_layer(ckpt, cfg, layer, rank, world)
                assert want.keys() == got.keys()
                for k in want:
                    assert torch.equal(want[k], got[k]), (world, rank, layer, k)
            want, got = tp.shard_head(sd, cfg, rank, world), tp.shard_head(ckpt, cfg, rank, world)
            for k in want:
                assert torch.equal(want[k], got[k]), (world, rank, k)


def test_interchange_with_the_safetensors_package(tmp_path):
    """Files written by the ``safetensors`` package (the format's own implementation, which the reference's crate
    follows) read back bit-exact through this reader, and files written here read back bit-exact through the package,
    for every dtype the reader maps, a zero-dimensional tensor, an empty tensor and the metadata block."""
    safetensors_torch = pytest.importorskip("safetensors.torch")
    from safetensors import safe_open
    from teenygrad_b200 import safetensors as st
    g = torch.Generator().manual_seed(3)
    tensors = {
        "model.layers.0.self_attn.q_proj.weight": torch.randn(48, 32, generator=g).bfloat16(),
        "model.norm.weight": torch.randn(32, generator=g).half(),
        "f32": torch.randn(3, 5, 7, generator=g),
        "f64": torch.randn(4, generator=g, dtype=torch.float64),
        "i64": torch.randint(-5, 5, (6,), generator=g),
        "i32": torch.randint(-5, 5, (2, 3), generator=g, dtype=torch.int32),
        "u8": torch.randint(0, 255, (9,), generator=g, dtype=torch.uint8),
        "flag": torch.tensor([True, False, True]),
        "scalar": torch.tensor(2.5),
        "empty": torch.zeros(0, 4),
    }
    theirs = tmp_path / "theirs.safetensors"
    safetensors_torch.save_file(tensors, str(theirs), metadata={"format": "pt"})
    mine = st.SafeTensors(theirs)
    assert sorted(mine) == sorted(tensors)
    for k, v in tensors.items():
        assert mine[k].dtype == v.dtype and tuple(mine[k].shape) == tuple(v.shape), k
        assert torch.equal(mine[k], v), k
    ours = tmp_path / "ours.safetensors"
    st.save_file(tensors, ours, metadata={"format": "pt"})
    back = safetensors_torch.load_file(str(ours))
    assert sorted(back) == sorted(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k], v), k
    with safe_open(str(ours), framework="pt") as f:
        assert f.metadata() == {"format": "pt"}
