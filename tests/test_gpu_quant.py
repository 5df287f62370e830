"""FP8 (E4M3) weight-only linear on the GPU against oracle/quant.py (the reference quantiser restated)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2  # bf16 bar of the path: max |got - want| / max |want|


@pytest.fixture(scope="module")
def ops():
    from teenygrad_b200 import ops as o
    return o


@pytest.fixture(autouse=True)
def _no_device_wait_errors(ops):
    yield
    assert ops.device_error(clear=True) == 0, "a kernel gave up on a bounded wait"


def rel(got, want):
    got, want = got.float().cpu(), torch.as_tensor(want).float()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def _case(M, N, K, strategy, group_size, seed=3):
    from oracle import quant as oq
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05 * (1 + 3 * torch.rand(N, 1, generator=g))).float().numpy()
    kw = {"tensor": {}, "channel": {"axis": 0}, "group": {"axis": 1, "group_size": group_size}}[strategy]
    q, s = oq.quantize_fp8(w, strategy, **kw)
    return x, q, s, kw


def test_dequant_every_byte_exact(ops):
    """All 256 encodings times a scale, one rounding to bf16: equal to the oracle bit for bit (NaN where it has NaN)."""
    from oracle import quant as oq
    q = np.tile(np.arange(256, dtype=np.uint8), (3, 1))
    s = np.array([1.0, 0.37, 2.0 ** -10], dtype=np.float32)
    want = torch.from_numpy(oq.dequantize_fp8(q, s, "channel", axis=0)).bfloat16()
    got = ops.dequant_fp8(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), "channel").cpu()
    nan = torch.isnan(want)
    assert torch.equal(torch.isnan(got), nan)
    assert torch.equal(got[~nan].view(torch.int16), want[~nan].view(torch.int16))
    assert ops.fp8_count_nan(torch.from_numpy(q).cuda()) == 6


@pytest.mark.parametrize("strategy,group_size", [("tensor", 0), ("channel", 0), ("group", 64), ("group", 128)])
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 512, 1024), (32, 4096, 4096), (7, 1000, 528), (64, 2048, 2048),
                                   (128, 1024, 4096), (33, 384, 2048), (5, 333, 1024), (4, 24576, 512)])
def test_linear_w8a16_small_m(ops, M, N, K, strategy, group_size):
    """The streaming path (bytes converted next to the tensor core): against the f32 dequantised weight, and equal
    run to run."""
    from oracle import quant as oq
    if strategy == "group" and K % group_size:
        pytest.skip("group size must divide K in this case list")
    x, q, s, kw = _case(M, N, K, strategy, group_size)
    want = oq.linear_w8a16(x.float().numpy(), q, s, strategy, **kw)
    qd, sd = torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda()
    first = None
    for _ in range(2):
        y = ops.linear_w8a16(x.cuda(), qd, sd, strategy, group_size)
        assert rel(y, want) < BF16_TOL
        first = y if first is None else first
        assert torch.equal(y, first)
    if strategy != "group":
        # scales applied to the f32 sums: as accurate as a bf16 GEMM over exact weights gets
        assert rel(y, want) < 8e-3


def test_linear_w8a16_subnormal_bytes_and_bias(ops):
    """Bytes the reference's quantiser never writes but its decoder reads (E4M3 subnormals), plus a bias."""
    from oracle import quant as oq
    rng = np.random.default_rng(5)
    q = rng.integers(0, 256, size=(256, 512), dtype=np.uint8)
    q[(q & 0x7F) == 0x7F] = 0x08                      # no NaN encodings
    q[:, ::3] &= 0x87                                 # a third of the columns: exponent 0 (subnormal or zero)
    s = (rng.random(256).astype(np.float32) + 0.5) * 1e-2
    x = (torch.randn(8, 512, generator=torch.Generator().manual_seed(6))).bfloat16()
    b = (torch.arange(256).float() * 0.01).bfloat16()
    want = oq.linear_w8a16(x.float().numpy(), q, s, "channel", axis=0, bias=b.float().numpy())
    y = ops.linear_w8a16(x.cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), "channel", bias=b.cuda())
    assert rel(y, want) < BF16_TOL


@pytest.mark.parametrize("strategy,group_size", [("channel", 0), ("group", 128)])
def test_linear_w8a16_large_m(ops, strategy, group_size):
    """M > 128: weight converted once into scratch (bf16(value * scale)), then the bf16 GEMM."""
    from oracle import quant as oq
    M, N, K = 300, 512, 1024
    x, q, s, kw = _case(M, N, K, strategy, group_size)
    want = oq.linear_w8a16(x.float().numpy(), q, s, strategy, **kw)
    y = ops.linear_w8a16(x.cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), strategy, group_size)
    assert rel(y, want) < BF16_TOL
    with pytest.raises(Exception):  # scratch too small is refused, not overrun
        ops.linear_w8a16(x.cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), strategy, group_size,
                         scratch=torch.empty(16, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("M,I,K", [(32, 3072, 1024), (4, 8192, 512), (128, 1024, 2048)])
def test_linear_w8a16_swiglu(ops, M, I, K):
    """Fused gate/up over interleaved FP8 rows equals the two projections through the oracle, then SwiGLU."""
    from oracle import cpu as oc
    from oracle import quant as oq
    g = torch.Generator().manual_seed(8)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    wg = (torch.randn(I, K, generator=g) * 0.05).float().numpy()
    wu = (torch.randn(I, K, generator=g) * 0.05).float().numpy()
    (qg, sg), (qu, su) = oq.quantize_fp8(wg, "channel", axis=0), oq.quantize_fp8(wu, "channel", axis=0)
    yg = torch.from_numpy(oq.linear_w8a16(x.float().numpy(), qg, sg, "channel", axis=0)).bfloat16()
    yu = torch.from_numpy(oq.linear_w8a16(x.float().numpy(), qu, su, "channel", axis=0)).bfloat16()
    want = oc.silu_mul_bf16(yg, yu)
    qi = ops.interleave_gate_up(torch.from_numpy(qg), torch.from_numpy(qu))
    si = ops.interleave_gate_up(torch.from_numpy(sg)[:, None], torch.from_numpy(su)[:, None])[:, 0].contiguous()
    out = ops.linear_w8a16(x.cuda(), qi.cuda(), si.cuda(), "channel", swiglu=True)
    assert rel(out, want) < BF16_TOL


def _check_generation(got_logits, got_ids, want_logits, want_ids):
    """Rows are comparable until their first token flip: logits within the bf16 bar up to there, and a flip must be a
    near-tie in the oracle's own logits (the chosen token within the bar of the best one)."""
    for i, g in enumerate(got_logits):
        same = (got_ids[:, :i] == want_ids[:, :i]).all(dim=1)
        if same.any():
            assert rel(g[same.cuda()], want_logits[same, i]) < BF16_TOL
        flipped = same & (got_ids[:, i] != want_ids[:, i])
        for b in torch.nonzero(flipped).flatten().tolist():
            row = want_logits[b, i].float()
            assert row.max() - row[got_ids[b, i]] < BF16_TOL * row.abs().max()
    assert (got_ids[:, 0] == want_ids[:, 0]).all()


def _quantized_checkpoint(ocfg, seed, strategy, group_size):
    """A random Qwen3 state dict quantised as the reference's quantiser does it (oracle/quant.py, its encoder restated):
    (tensors as they go into the file, metadata, state dict of the dequantised float32 weights)."""
    import json

    from oracle import quant as oq
    from oracle import qwen3 as oqw
    sd = oqw.make_weights(ocfg, seed)
    kw = {"tensor": {}, "channel": {"axis": 0}, "group": {"axis": 1, "group_size": group_size}}[strategy]
    tensors, deq, ignore = {}, {}, []
    for name, t in sd.items():
        if t.dim() >= 2:
            q, s = oq.quantize_fp8(t.float().numpy(), strategy, **kw)
            tensors[name] = torch.from_numpy(q).view(torch.float8_e4m3fn)
            tensors[name + "_scale"] = torch.from_numpy(s)
            deq[name] = torch.from_numpy(oq.dequantize_fp8(q, s, strategy, **kw))
        else:
            tensors[name] = t
            deq[name] = t
            ignore.append(name)
    weights = dict(num_bits=8, type="float", symmetric=True, strategy=strategy, fp8_variant="e4m3", **kw)
    meta = {"quantization_config": json.dumps({
        "quant_method": "compressed-tensors", "format": "float-quantized",
        "config_groups": {"group_0": {"weights": weights, "targets": ["*"]}}, "ignore": ignore})}
    return tensors, meta, deq


@pytest.mark.parametrize("strategy,group_size,B,S", [("channel", 0, 3, 40), ("group", 128, 2, 200), ("tensor", 0, 2, 24)])
def test_runner_on_a_float_quantized_checkpoint(tmp_path, strategy, group_size, B, S):
    """File written in the reference quantiser's layout -> reader -> runner with FP8 projections and LM head, against
    the CPU oracle run on the dequantised weights (bf16 activations times f32 weights, rounded to bf16 per linear).
    S = 200 exercises the prefill path that converts a projection into scratch, the others the streaming path."""
    from oracle import qwen3 as oqw
    from teenygrad_b200 import qwen3, quant
    from teenygrad_b200 import safetensors as st
    ocfg = oqw.OracleQwen3Config(3, 512, 8, 2, 128, 1024, 4096, tied=False)
    tensors, meta, deq = _quantized_checkpoint(ocfg, 11, strategy, group_size)
    st.save_file(tensors, tmp_path / "model.safetensors", metadata=meta)
    ck = st.SafeTensors(tmp_path / "model.safetensors")
    scheme, ignore = quant.parse_quantization_config(ck.metadata)
    assert scheme.strategy == strategy and scheme.group_size == group_size and "model.norm.weight" in ignore
    steps = 10
    ids = torch.randint(0, ocfg.vocab, (B, S), generator=torch.Generator().manual_seed(12))
    deq["model.embed_tokens.weight"] = deq["model.embed_tokens.weight"].bfloat16()  # the lookup table is stored as bf16
    want_ids, want_logits = oqw.OracleQwen3(ocfg, deq, f32_twin=True).generate(ids, steps, return_logits=True)
    cfg = qwen3.Qwen3Config(3, 512, 8, 2, 128, 1024, 4096, tied=False)
    r = qwen3.Qwen3Runner(cfg, max_batch=B, max_len=S + steps, max_new_tokens=steps)
    r.load_quantized({k: ck[k] for k in ck}, scheme)
    r.prefill(ids)
    got = [r.logits().clone()]
    for _ in range(steps - 1):
        r.decode_step(graph=True)
        got.append(r.logits().clone())
    assert qwen3.lib.teeny_device_error(1) == 0
    got_ids = r.history()[:steps].t().cpu().long()
    _check_generation(got, got_ids, want_logits, want_ids)


@pytest.mark.parametrize("bits,symmetric,strategy,group_size", [(8, True, "channel", 0), (8, False, "tensor", 0),
                                                                (4, True, "group", 32), (4, False, "channel", 0)])
def test_dequant_int_equals_the_oracle(ops, bits, symmetric, strategy, group_size):
    """Integer schemes (int8, nibble-packed int4; symmetric and with zero points): bit-equal to the oracle's
    dequantisation rounded once to bf16.  Odd K puts rows on nibble boundaries inside a byte."""
    from oracle import quant as oq
    rng = np.random.default_rng(7)
    N, K = 37, 75
    w = (rng.standard_normal((N, K)) * 0.1 + 0.03).astype(np.float32)
    kw = {"tensor": {}, "channel": {"axis": 0}, "group": {"axis": 1, "group_size": group_size}}[strategy]
    q, s, zp = oq.quantize_affine(w, bits, symmetric, strategy, **kw)
    want = torch.from_numpy(oq.dequantize_affine(q, s, zp, strategy, **kw)).bfloat16()
    stored = torch.from_numpy(q) if bits == 8 else torch.from_numpy(oq.pack_i4(q))
    got = ops.dequant_int(stored.cuda(), bits, torch.from_numpy(s).cuda(), None if symmetric else torch.from_numpy(zp).cuda(),
                          (N, K), strategy, group_size)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


def test_runner_on_a_pack_quantized_int4_checkpoint(tmp_path):
    """4-bit checkpoint in the quantiser's layout (packed U8 vectors, logical shapes in the metadata) -> reader ->
    runner (weights converted to bf16 at load) against the CPU oracle on the same dequantised bf16 weights."""
    import json

    from oracle import quant as oq
    from oracle import qwen3 as oqw
    from teenygrad_b200 import qwen3, quant
    from teenygrad_b200 import safetensors as st
    ocfg = oqw.OracleQwen3Config(2, 256, 4, 2, 128, 512, 1024, tied=False)
    sd = oqw.make_weights(ocfg, 21)
    tensors, deq, shapes, ignore = {}, {}, {}, []
    for name, t in sd.items():
        if t.dim() >= 2:
            q, s, zp = oq.quantize_affine(t.float().numpy(), 4, False, "group", axis=1, group_size=64)
            tensors[name] = torch.from_numpy(oq.pack_i4(q))
            tensors[name + "_scale"] = torch.from_numpy(s)
            tensors[name + "_zero_point"] = torch.from_numpy(zp)
            shapes[name] = {"logical_shape": list(t.shape), "elements": t.numel()}
            deq[name] = torch.from_numpy(oq.dequantize_affine(q, s, zp, "group", axis=1, group_size=64)).bfloat16()
        else:
            tensors[name] = t
            deq[name] = t
            ignore.append(name)
    weights = dict(num_bits=4, type="int", symmetric=False, strategy="group", axis=1, group_size=64)
    meta = {"quantization_config": json.dumps({
        "quant_method": "compressed-tensors", "format": "pack-quantized",
        "config_groups": {"group_0": {"weights": weights, "targets": ["*"]}}, "ignore": ignore,
        "teenygrad_packed_int4": shapes})}
    st.save_file(tensors, tmp_path / "model.safetensors", metadata=meta)
    ck = st.SafeTensors(tmp_path / "model.safetensors")
    scheme, _ = quant.parse_quantization_config(ck.metadata)
    assert isinstance(scheme, quant.IntScheme) and scheme.bits == 4 and not scheme.symmetric
    B, S, steps = 2, 24, 8
    ids = torch.randint(0, ocfg.vocab, (B, S), generator=torch.Generator().manual_seed(22))
    want_ids, want_logits = oqw.OracleQwen3(ocfg, deq).generate(ids, steps, return_logits=True)
    r = qwen3.Qwen3Runner(qwen3.Qwen3Config(2, 256, 4, 2, 128, 512, 1024, tied=False), max_batch=B, max_len=S + steps,
                          max_new_tokens=steps)
    r.load_quantized({k: ck[k] for k in ck}, scheme)
    r.prefill(ids)
    got = [r.logits().clone()]
    for _ in range(steps - 1):
        r.decode_step(graph=True)
        got.append(r.logits().clone())
    _check_generation(got, r.history()[:steps].t().cpu().long(), want_logits, want_ids)


@pytest.mark.parametrize("M,K", [(37, 1000), (37, 1003), (32, 12288)])   # 16-byte pieces / a ragged row / the MLP width
def test_split_fp8_equals_the_oracle_split(ops, M, K):
    """The two-term E4M3 split of bf16 activations: bytes and scales equal to the oracle's, bit for bit."""
    from oracle import quant as oq
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(M, K, generator=g) * torch.logspace(-3, 3, M)[:, None]).bfloat16()
    x[4] = 0
    x[9, ::3] *= 1e-4                      # elements far below their row's maximum
    hi, lo, inv_s = oq.split_e4m3(x.float().numpy())
    out, scale = ops.split_fp8(x.cuda())
    assert torch.equal(out[:M].cpu(), torch.from_numpy(hi)) and torch.equal(out[M:].cpu(), torch.from_numpy(lo))
    assert torch.equal(scale.cpu(), torch.from_numpy(inv_s))


@pytest.mark.parametrize("strategy", ["tensor", "channel"])
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 512, 1024), (32, 4096, 4096), (7, 1000, 528), (64, 2048, 2048),
                                   (128, 1024, 4096), (5, 333, 1024), (4, 24576, 512), (32, 4096, 12288)])
def test_linear_w8a8x2(ops, M, N, K, strategy):
    """FP8 weights x two-term FP8 activations (kind::f8f6f4, nothing converted in the kernel): equal to the oracle
    evaluated on the split activations, and -- the split being exact for all but tiny elements -- to the weight-only
    result on the bf16 activations themselves."""
    from oracle import quant as oq
    x, q, s, kw = _case(M, N, K, strategy, 0)
    hi, lo, inv_s = oq.split_e4m3(x.float().numpy())
    want_split = oq.linear_w8a8x2(hi, lo, inv_s, q, s, strategy, **kw)
    want_exact = oq.linear_w8a16(x.float().numpy(), q, s, strategy, **kw)
    x8, xs = ops.split_fp8(x.cuda())
    qd, sd = torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda()
    first = None
    for _ in range(2):
        y = ops.linear_w8a8x2(x8, xs, qd, sd, strategy)
        assert rel(y, want_split) < 8e-3 and rel(y, want_exact) < 8e-3
        first = y if first is None else first
        assert torch.equal(y, first)


def test_linear_w8a8x2_swiglu_and_bias(ops):
    from oracle import cpu as oc
    from oracle import quant as oq
    M, I, K = 32, 3072, 1024
    g = torch.Generator().manual_seed(33)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    wg = (torch.randn(I, K, generator=g) * 0.05).float().numpy()
    wu = (torch.randn(I, K, generator=g) * 0.05).float().numpy()
    (qg, sg), (qu, su) = oq.quantize_fp8(wg, "channel", axis=0), oq.quantize_fp8(wu, "channel", axis=0)
    yg = torch.from_numpy(oq.linear_w8a16(x.float().numpy(), qg, sg, "channel", axis=0)).bfloat16()
    yu = torch.from_numpy(oq.linear_w8a16(x.float().numpy(), qu, su, "channel", axis=0)).bfloat16()
    qi = ops.interleave_gate_up(torch.from_numpy(qg), torch.from_numpy(qu))
    si = ops.interleave_gate_up(torch.from_numpy(sg)[:, None], torch.from_numpy(su)[:, None])[:, 0].contiguous()
    x8, xs = ops.split_fp8(x.cuda())
    out = ops.linear_w8a8x2(x8, xs, qi.cuda(), si.cuda(), "channel", swiglu=True)
    assert rel(out, oc.silu_mul_bf16(yg, yu)) < BF16_TOL
    b = (torch.arange(I).float() * 0.01).bfloat16()
    yb = ops.linear_w8a8x2(x8, xs, torch.from_numpy(qg).cuda(), torch.from_numpy(sg).cuda(), "channel", bias=b.cuda())
    assert rel(yb, oq.linear_w8a16(x.float().numpy(), qg, sg, "channel", axis=0, bias=b.float().numpy())) < BF16_TOL
