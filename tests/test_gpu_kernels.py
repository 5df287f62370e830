"""GPU parity tests: every C-ABI kernel against the CPU oracle on the same seeded inputs.

Bars (BASELINE north_star): f32 outputs within 1e-4, bf16 within 2e-2, both measured as
max|a - e| / max|e| over the tensor; the reference's own per-element bounds are asserted where its tests
state one.  Integer results (argmax, gathered rows) must be bit exact.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
F32_TOL = 1e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from teenygrad_b200 import ops as o
    return o


@pytest.fixture(autouse=True)
def _no_device_wait_errors(ops):
    yield
    assert ops.device_error(clear=True) == 0, "a kernel gave up on a bounded wait"


def rel(a, e):
    a, e = a.detach().float().cpu(), e.detach().float().cpu()
    return float((a - e).abs().max() / e.abs().max().clamp_min(1e-30))


def dev(x):
    return torch.as_tensor(x).cuda()


# ---------------------------------------------------------------------------------------------- f32, fixtures
def test_matmul_f32_ramp_fixture(ops, golden):
    c = ops.matmul_forward(dev(golden["gemm_ramp_a"]), dev(golden["gemm_ramp_b"]))
    e = torch.from_numpy(golden["gemm_ramp_expected"])
    assert rel(c, e) < F32_TOL
    assert torch.all((c.cpu() - e).abs() < 1e-2 + 1e-3 * e.abs())  # test_gemm.rs:41-47


def test_matmul_f32_512_config(ops):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(512, 512, generator=g), torch.randn(512, 512, generator=g)
    c = ops.matmul_forward(a.cuda(), b.cuda())
    assert rel(c, torch.from_numpy(oc.matmul_f32(a.numpy(), b.numpy()))) < F32_TOL


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (128, 136, 72), (300, 264, 200), (1024, 2048, 512), (5, 8, 8)])
def test_matmul_f32_on_tensor_cores_keeps_f32_accuracy(ops, M, N, K):
    """With scratch the f32 matmul runs as one bf16 GEMM over operands split into two bf16 terms (three products): the
    1e-4 bar must hold with a wide margin (a single reduced-precision pass would sit near 1e-3)."""
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(M + N + K)
    a, b = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)
    a[0, 0], b[0, 0] = 1000.0, -1000.0   # a large product next to ordinary ones
    e = torch.from_numpy(oc.matmul_f32(a.numpy(), b.numpy()))
    c = ops.matmul_forward(a.cuda(), b.cuda(), scratch=ops.matmul_f32_scratch(M, N, K))
    assert rel(c, e) < 2e-5
    c_simt = ops.matmul_forward(a.cuda(), b.cuda())
    assert rel(c_simt, e) < F32_TOL


def test_matmul_f32_ramp_fixture_on_tensor_cores(ops, golden):
    a, b = dev(golden["gemm_ramp_a"]), dev(golden["gemm_ramp_b"])
    M, K = a.shape
    N = b.shape[1]
    if K % 8 or N % 8:
        pytest.skip("fixture shape is not a multiple of 8: served by the CUDA-core kernel")
    c = ops.matmul_forward(a, b, scratch=ops.matmul_f32_scratch(M, N, K))
    e = torch.from_numpy(golden["gemm_ramp_expected"])
    assert rel(c, e) < F32_TOL
    assert torch.all((c.cpu() - e).abs() < 1e-2 + 1e-3 * e.abs())  # test_gemm.rs:41-47


def test_linear_f32_fixture(ops, golden):
    x, w, b = dev(golden["linear_input"]), dev(golden["linear_weight"]), dev(golden["linear_bias"])
    assert rel(ops.linear_forward(x, w), torch.from_numpy(golden["linear_expected_no_bias"])) < F32_TOL
    assert rel(ops.linear_forward(x, w, b), torch.from_numpy(golden["linear_expected_with_bias"])) < F32_TOL


def test_flash_attn2_f32_fixture(ops, golden):
    o, l = ops.flash_attention2_forward(dev(golden["fa2_q"]), dev(golden["fa2_k"]), dev(golden["fa2_v"]), 0.125)
    assert np.abs(o.cpu().numpy() - golden["fa2_expected_forward_o"]).max() < 1e-4  # test_flash_attn2.rs:152-168
    assert np.abs(l.cpu().numpy() - golden["fa2_expected_forward_l"]).max() < 1e-4


def test_rmsnorm_f32_fixture(ops, golden):
    y, rrms = ops.rms_norm_forward(dev(golden["rmsnorm_x"]), dev(golden["rmsnorm_weight"]), 1e-8, want_rrms=True)
    assert np.abs(y.cpu().numpy() - golden["rmsnorm_expected_forward"]).max() < 1e-4
    assert np.abs(rrms.cpu().numpy() - golden["rmsnorm_expected_rrms"]).max() < 1e-4


def test_elementwise_f32_fixtures(ops, golden):
    assert np.abs(ops.silu_forward(dev(golden["silu_x"])).cpu().numpy() - golden["silu_expected_forward"]).max() < 1e-5
    a, b = dev(golden["binary_a"]), dev(golden["binary_b"])
    assert np.array_equal(ops.elemwise_mul_forward(a, b).cpu().numpy(), golden["binary_expected_mul"])
    assert np.array_equal(ops.elemwise_add_forward(a, b).cpu().numpy(), golden["binary_expected_sum"])
    assert np.array_equal(ops.elemwise_add_forward(dev(golden["add_a"]), dev(golden["add_b"])).cpu().numpy(),
                          golden["add_expected_fwd"])
    y = ops.softmax_forward(dev(golden["softmax_x_forward"]))
    assert np.abs(y.cpu().numpy() - golden["softmax_expected_forward"]).max() < 1e-6


def test_elementwise_ragged_sizes(ops):
    g = torch.Generator().manual_seed(5)
    for n in (1, 7, 1023, 4097):
        a, b = torch.randn(n, generator=g), torch.randn(n, generator=g)
        assert torch.equal(ops.elemwise_add_forward(a.cuda(), b.cuda()).cpu(), a + b)
        ab, bb = a.bfloat16(), b.bfloat16()
        assert torch.equal(ops.elemwise_mul_forward(ab.cuda(), bb.cuda()).cpu(), ab * bb)
        assert torch.equal(ops.elemwise_add_forward(ab.cuda(), bb.cuda()).cpu(), ab + bb)


# ---------------------------------------------------------------------------------------------- bf16 GEMM
def _gemm_inputs(M, N, K, seed=1):
    g = torch.Generator().manual_seed(seed)
    x = ((torch.rand(M, K, generator=g) * 2 - 1) * 0.05).bfloat16()
    w = ((torch.rand(N, K, generator=g) * 2 - 1) * 0.05).bfloat16()
    return x, w


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 64), (128, 128, 128), (256, 512, 512), (300, 200, 136), (4096, 512, 256), (129, 264, 72),
    (1024, 1024, 1024), (4096, 4096, 512), (2500, 5000, 264), (8192, 2304, 1088),
])
def test_linear_bf16_large_m(ops, M, N, K):
    from oracle import cpu as oc
    x, w = _gemm_inputs(M, N, K)
    y = ops.linear_forward(x.cuda(), w.cuda())
    assert rel(y, oc.linear_bf16(x, w)) < BF16_TOL


@pytest.mark.parametrize("M,N,K", [
    (1, 256, 512), (16, 512, 1024), (32, 4096, 4096), (1, 4096, 4096), (7, 1000, 520), (64, 2048, 2048),
    (128, 1024, 4096), (33, 384, 2048), (5, 333, 1024), (100, 130, 4096), (3, 6, 2048), (13, 4097, 512),
    # BASELINE config 2 at its exact shapes: N = K = 4096 with M = 1, 16, 128
    (16, 4096, 4096), (128, 4096, 4096),
])
def test_linear_bf16_small_m_cluster_splitk(ops, M, N, K):
    """M <= 128: weights on the 128-row side of the MMA, K split over a thread-block cluster and summed through
    distributed shared memory (no global scratch; the entry point's scratch argument stays NULL)."""
    from oracle import cpu as oc
    x, w = _gemm_inputs(M, N, K)
    e = oc.linear_bf16(x, w)
    assert ops.lib.teeny_gemm_scratch_bytes(M, N, K) == 0
    first = None
    for _ in range(2):  # deterministic: the cluster sums its partial tiles in rank order
        y = ops.linear_forward(x.cuda(), w.cuda())
        assert rel(y, e) < BF16_TOL
        first = y if first is None else first
        assert torch.equal(y, first)


def test_linear_bf16_bias_and_strided_fallback(ops):
    from oracle import cpu as oc
    x, w = _gemm_inputs(200, 136, 264)
    b = (torch.arange(136).float() * 0.01).bfloat16()
    assert rel(ops.linear_forward(x.cuda(), w.cuda(), b.cuda()), oc.linear_bf16(x, w, b)) < BF16_TOL
    xs, ws = _gemm_inputs(16, 256, 512)
    assert rel(ops.linear_forward(xs.cuda(), ws.cuda(), (torch.arange(256).float() * 0.01).bfloat16().cuda()),
               oc.linear_bf16(xs, ws, (torch.arange(256).float() * 0.01).bfloat16())) < BF16_TOL
    xt = x.cuda().t().contiguous().t()  # column-major view: takes the CUDA-core kernel
    assert rel(ops.linear_forward(xt, w.cuda()), oc.linear_bf16(x, w)) < BF16_TOL
    x2, w2 = _gemm_inputs(9, 10, 11)     # K not a multiple of 8
    assert rel(ops.linear_forward(x2.cuda(), w2.cuda()), oc.linear_bf16(x2, w2)) < BF16_TOL


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 320, 192), (100, 72, 40), (512, 1024, 512)])
def test_matmul_bf16_row_major_b(ops, M, N, K):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(7)
    a = ((torch.rand(M, K, generator=g) * 2 - 1) * 0.05).bfloat16()
    b = ((torch.rand(K, N, generator=g) * 2 - 1) * 0.05).bfloat16()
    assert rel(ops.matmul_forward(a.cuda(), b.cuda()), oc.matmul_bf16(a, b)) < BF16_TOL


def test_linear_bf16_linearity_full_size(ops):
    """Config-2 size (M=4096, N=K=4096): too slow for the CPU oracle in a test, so check structure:
    rows of Y depend only on the matching rows of X, and a one-hot X row reads back a row of W^T."""
    x, w = _gemm_inputs(4096, 4096, 4096)
    xc, wc = x.cuda(), w.cuda()
    y = ops.linear_forward(xc, wc)
    y_top = ops.linear_forward(xc[:128].contiguous(), wc)
    assert rel(y[:128], y_top) < 5e-3  # same products; only the accumulation grouping may differ
    onehot = torch.zeros(128, 4096, dtype=torch.bfloat16)
    onehot[torch.arange(128), torch.arange(128) * 31] = 1.0
    sel = ops.linear_forward(onehot.cuda(), wc)
    assert torch.equal(sel.cpu(), w[:, torch.arange(128) * 31].t().contiguous())
    from oracle import cpu as oc
    rows = torch.tensor([0, 1, 127, 128, 2047, 4095])
    assert rel(y[rows.cuda()], oc.linear_bf16(x[rows], w)) < BF16_TOL


# ---------------------------------------------------------------------------------------------- attention
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (1, 1, 1, 128, 128, True), (1, 4, 1, 256, 256, True), (2, 4, 2, 384, 384, True), (1, 2, 2, 200, 200, True),
    (1, 2, 1, 128, 512, True), (1, 2, 1, 130, 300, False), (1, 8, 2, 1024, 1024, True),
])
def test_flash_attn_prefill_bf16(ops, B, Hq, Hkv, Sq, Skv, causal):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(2)
    q = torch.randn(B, Hq, Sq, 128, generator=g).bfloat16()
    k = torch.randn(B, Hkv, Skv, 128, generator=g).bfloat16()
    v = torch.randn(B, Hkv, Skv, 128, generator=g).bfloat16()
    o, lse = ops.flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, causal=causal, want_lse=True)
    eo, el = oc.attention_bf16(q, k, v, 128 ** -0.5, causal=causal)
    assert rel(o, eo) < BF16_TOL
    assert (lse.cpu() - el).abs().max() < 2e-2


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (16, 32, 8, 256, 256, True),    # 512 items of two key tiles each: every CTA pair walks several short items in a row
    (8, 32, 8, 640, 640, True),     # 2, 4 and 5 key tiles: the softmax group that finishes an item alternates
    (4, 32, 8, 300, 900, False),    # ragged query tile, eight key tiles per item
    (24, 16, 4, 100, 100, True),    # one key tile per item
    (8, 32, 8, 200, 712, True),     # queries at the end of a longer history (query i sees keys <= i + 512), six key tiles
])
def test_flash_attn_prefill_many_items_per_cta_pair(ops, B, Hq, Hkv, Sq, Skv, causal):
    """More (query tile, head, batch) items than CTA pairs, so that one item's output overlaps the next item's start."""
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, Hq, Sq, 128, generator=g).bfloat16()
    k = torch.randn(B, Hkv, Skv, 128, generator=g).bfloat16()
    v = torch.randn(B, Hkv, Skv, 128, generator=g).bfloat16()
    o, lse = ops.flash_attn_fwd(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, causal=causal, want_lse=True)
    assert ops.device_error() == 0
    eo, el = oc.attention_bf16(q, k, v, 128 ** -0.5, causal=causal)
    assert rel(o, eo) < BF16_TOL
    assert (lse.cpu() - el).abs().max() < 2e-2
    # per (batch, head) as well: a mixed-up item would vanish in the norm over the whole tensor
    per = ((o.cpu().float() - eo.float()).flatten(2).norm(dim=2) / eo.float().flatten(2).norm(dim=2)).max()
    assert per < BF16_TOL


def test_flash_attn_token_major_views(ops):
    """The layout the Qwen3 runner uses: q inside a fused [T, (Hq+2Hkv)*D] projection, output [B, S, Hq*D]."""
    from oracle import cpu as oc
    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).bfloat16().cuda()
    q = qkv[:, :Hq * D].view(B, S, Hq, D).permute(0, 2, 1, 3)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D).permute(0, 2, 1, 3)
    v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D).permute(0, 2, 1, 3)
    out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device="cuda")
    ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, out=out.permute(0, 2, 1, 3))
    eo, _ = oc.attention_bf16(q.cpu(), k.cpu(), v.cpu(), D ** -0.5, causal=True)
    assert rel(out.permute(0, 2, 1, 3), eo) < BF16_TOL


def test_flash_attn2_bf16_reference_layout(ops):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(3, 160, 128, generator=g).bfloat16() for _ in range(3))
    o, l = ops.flash_attention2_forward(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5)
    eo, el = oc.attention_bf16(q[None], k[None], v[None], 128 ** -0.5, causal=False)
    assert rel(o, eo[0]) < BF16_TOL and (l.cpu() - el[0]).abs().max() < 2e-2
    q, k, v = (torch.randn(2, 9, 64, generator=g).bfloat16() for _ in range(3))  # head_dim 64: CUDA-core kernel
    o, _ = ops.flash_attention2_forward(q.cuda(), k.cuda(), v.cuda(), 0.125)
    eo, _ = oc.attention_bf16(q[None], k[None], v[None], 0.125, causal=False)
    assert rel(o, eo[0]) < BF16_TOL


@pytest.mark.parametrize("B,Hq,Hkv,cap,L", [(2, 8, 2, 1024, 1024), (1, 4, 1, 2048, 700), (3, 16, 8, 640, 1),
                                            (2, 32, 8, 4096, 4096), (1, 2, 2, 600, 513), (2, 8, 1, 512, 37)])
def test_flash_attn_decode_bf16(ops, B, Hq, Hkv, cap, L):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(2)
    q = torch.randn(B, Hq, 1, 128, generator=g).bfloat16()
    k = torch.randn(B, Hkv, cap, 128, generator=g).bfloat16()
    v = torch.randn(B, Hkv, cap, 128, generator=g).bfloat16()
    eo, _ = oc.attention_bf16(q, k[:, :, :L], v[:, :, :L], 128 ** -0.5, causal=False)
    kc, vc = k.cuda(), v.cuda()
    kc[:, :, L:] = float("nan")  # rows past the live length must never be read into the result
    vc[:, :, L:] = float("nan")
    o = ops.flash_attn_decode(q.cuda(), kc, vc, L, 128 ** -0.5)
    assert rel(o, eo) < BF16_TOL
    o2 = ops.flash_attn_decode(q.cuda(), kc, vc, torch.tensor([L], dtype=torch.int32, device="cuda"), 128 ** -0.5)
    assert torch.equal(o, o2)


# ---------------------------------------------------------------------------------------------- norms & fused
@pytest.mark.parametrize("M,N", [(5, 1024), (33, 4096), (64, 128), (3, 8192), (4, 1000), (2, 12288)])
def test_rms_norm_bf16(ops, M, N):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, N, generator=g).bfloat16()
    w = (torch.rand(N, generator=g) + 0.5).bfloat16()
    y = ops.rms_norm_forward(x.cuda(), w.cuda(), 1e-6)
    e = oc.rms_norm_bf16(x, w, 1e-6)
    assert rel(y, e) < BF16_TOL
    assert (y.cpu() != e).float().mean() < 0.01  # same rounding points: all but rare half-ulp cases identical


def test_add_rms_norm_bf16(ops):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(8)
    x, r = torch.randn(40, 4096, generator=g).bfloat16(), torch.randn(40, 4096, generator=g).bfloat16()
    w = (torch.rand(4096, generator=g) + 0.5).bfloat16()
    rc = r.cuda()
    y = ops.add_rms_norm(x.cuda(), rc, w.cuda(), 1e-6)
    h = r + x
    assert torch.equal(rc.cpu(), h)
    assert rel(y, oc.rms_norm_bf16(h, w, 1e-6)) < BF16_TOL


def test_silu_mul_bf16(ops):
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(9)
    gu = torch.randn(37, 2 * 3072, generator=g).bfloat16()
    out = ops.silu_mul(gu.cuda())
    e = oc.silu_mul_bf16(gu[:, :3072], gu[:, 3072:])
    assert rel(out, e) < BF16_TOL
    assert (out.cpu() != e).float().mean() < 0.01


@pytest.mark.parametrize("M,I,K", [(32, 3072, 1024), (1, 128, 512), (7, 1536, 4096), (300, 1024, 512), (4096, 3072, 1024),
                                   (128, 12288, 4096), (129, 640, 264), (8192, 3072, 512), (5000, 2496, 264),
                                   (4, 8192, 512)])  # the last: one CTA per weight tile, no cluster

def test_linear_swiglu_fused(ops, M, I, K):
    """One GEMM over interleaved gate/up rows must equal linear -> linear -> silu -> mul of the bf16 graph."""
    from oracle import cpu as oc
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    wg = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(I, K, generator=g) * 0.05).bfloat16()
    out = ops.linear_swiglu(x.cuda(), ops.interleave_gate_up(wg, wu).cuda())
    e = oc.silu_mul_bf16(oc.linear_bf16(x, wg), oc.linear_bf16(x, wu))
    assert rel(out, e) < BF16_TOL
    # and against this library's own unfused kernels: same rounding points, so nearly every element is identical
    gu = ops.linear_forward(x.cuda(), torch.cat([wg, wu]).cuda())
    unfused = ops.silu_mul(gu)
    assert (out != unfused).float().mean() < 0.02 and rel(out, unfused) < BF16_TOL


def test_embedding_and_argmax_exact(ops):
    g = torch.Generator().manual_seed(10)
    table = torch.randn(1000, 256, generator=g).bfloat16()
    ids = torch.randint(0, 1000, (77,), generator=g, dtype=torch.int32)
    assert torch.equal(ops.embedding(ids.cuda(), table.cuda()).cpu(), table[ids.long()])
    logits = torch.randn(5, 151936, generator=g).bfloat16()
    logits[2, 70000] = logits[2, 140000] = 9.0  # tie: lowest index wins
    val, idx = ops.argmax(logits.cuda())
    assert torch.equal(idx.cpu().long(), torch.argmax(logits.float(), dim=-1))
    assert int(idx[2]) == 70000
    # vocabulary split over 4 parts, then merged
    parts = [ops.argmax(logits[:, i * 37984:(i + 1) * 37984].contiguous().cuda(), idx_offset=i * 37984) for i in range(4)]
    merged = ops.argmax_combine(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert torch.equal(merged.cpu(), idx.cpu())


def test_rope_table_and_qk_norm_rope_kv(ops):
    from oracle import qwen3 as oq
    from oracle import cpu as oc
    cfg = oq.OracleQwen3Config(1, 512, 4, 2, 128, 512, 100)
    max_len, B, S, pos0 = 64, 2, 5, 7
    cos, sin = ops.rope_table(oq.inv_freq(cfg).cuda(), max_len)
    ec, es = oq.rope_tables(cfg, torch.arange(max_len))
    assert (cos.cpu() != ec).float().mean() < 1e-3 and (sin.cpu() != es).float().mean() < 1e-3
    assert rel(cos, ec) < 1e-2 and rel(sin, es) < 1e-2
    g = torch.Generator().manual_seed(11)
    Hq, Hkv, D = 4, 2, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    qw, kw = (torch.rand(D, generator=g) + 0.5).bfloat16(), (torch.rand(D, generator=g) + 0.5).bfloat16()
    kc = torch.zeros(B, Hkv, max_len, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qkv_d = qkv.cuda()
    ops.qk_norm_rope_kv(qkv_d, qw.cuda(), kw.cuda(), cos, sin, kc, vc, S, Hq, Hkv, pos0, 1e-6)
    q = qkv[:, :Hq * D].view(B, S, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
    c, s_ = ec[pos0:pos0 + S][None, :, None], es[pos0:pos0 + S][None, :, None]
    qn, kn = oc.rms_norm_bf16(q, qw, 1e-6), oc.rms_norm_bf16(k, kw, 1e-6)
    eq = qn * c + oq._rotate_half(qn) * s_
    ek = kn * c + oq._rotate_half(kn) * s_
    got_q = qkv_d[:, :Hq * D].view(B, S, Hq, D).cpu()
    assert rel(got_q, eq) < BF16_TOL and (got_q != eq).float().mean() < 0.01
    assert rel(kc[:, :, pos0:pos0 + S].cpu(), ek.transpose(1, 2)) < BF16_TOL
    assert torch.equal(vc[:, :, pos0:pos0 + S].cpu(), v.transpose(1, 2))
    assert float(kc[:, :, :pos0].abs().sum()) == 0 and float(kc[:, :, pos0 + S:].abs().sum()) == 0


# ---------------------------------------------------------------------------------------------------------------
# sampling behind the LM head
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,temperature,top_k,top_p", [
    (4, 1000, 1.0, 1, 1.0),          # top-k 1 = argmax
    (8, 151936, 0.8, 50, 0.9),       # Qwen3 vocabulary, usual serving settings
    (3, 151936, 1.5, 1024, 0.95),    # widest candidate list
    (5, 777, 0.3, 1024, 1.0),        # fewer columns than top_k, odd row length
    (6, 32000, 1.0, 40, 0.5),
])
def test_sample_top_k_top_p_matches_oracle(ops, rows, cols, temperature, top_k, top_p):
    from oracle import sampling as osamp
    g = torch.Generator().manual_seed(rows * 131 + cols)
    logits = (torch.randn(rows, cols, generator=g) * 3).bfloat16()
    if top_k == 1:
        logits[0, [5, 9, 700]] = 20.0  # ties at the top: the lowest index must win
    u = torch.rand(rows, generator=g)
    got, prob = ops.sample_top_k_top_p(logits.cuda(), temperature, top_k, top_p, u.cuda(), want_prob=True)
    got, prob = got.cpu().numpy(), prob.cpu().numpy()
    lf = logits.float().numpy()
    for r in range(rows):
        want, wprob, c, n, cand = osamp.sample_row(lf[r], temperature, top_k, top_p, float(u[r]))
        if got[r] == want:
            assert abs(prob[r] - wprob) <= 1e-4 * max(1.0, wprob)
            continue
        # exp() differs by a few ulp between the GPU and numpy, so at a boundary of the CDF the neighbour may be
        # picked: accept only a candidate of the nucleus (or the first one past it) whose CDF interval lies within
        # 1e-5 (relative) of u
        cl = list(cand)
        assert got[r] in cl[:n + 1], f"row {r}: {got[r]} is not a nucleus candidate"
        i = cl.index(got[r])
        lo = c[i - 1] if i > 0 else 0.0
        target = np.float32(u[r]) * c[n - 1]
        tol = 1e-5 * c[n - 1]
        assert lo - tol <= target <= c[i] + tol, f"row {r}: picked {got[r]} outside its CDF interval"
    assert ops.device_error() == 0


# ---------------------------------------------------------------------------------------------------------------
# the receiving half of the tensor-parallel decode reduction, with the ranks' pushes laid out by the test
# ---------------------------------------------------------------------------------------------------------------
def _stamped(values_f32, stamp):
    """[..., N] f32 -> [..., N] 64-bit words {value bits, stamp} as the GEMM push epilogue stores them."""
    bits = values_f32.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return bits | (int(stamp) << 32)


@pytest.mark.parametrize("world,M,N", [(2, 5, 1024), (4, 32, 4096), (8, 32, 4096), (3, 7, 8192)])
def test_tp_gather_add_rms_norm_sums_stamped_partials(ops, world, M, N):
    import ctypes as C
    from oracle import cpu as oc
    from teenygrad_b200 import qwen3
    g = torch.Generator().manual_seed(world * 100 + M)
    parts = torch.randn(world, M, N, generator=g) * 0.1
    res = torch.randn(M, N, generator=g).bfloat16()
    w = (torch.rand(N, generator=g) + 0.5).bfloat16()
    epoch, rnd = 37, 5
    stamp = epoch * 1024 + rnd + 1
    rows_cap = M + 3                      # slots are sized for the runner's max batch, not for this call
    recv = torch.zeros(world, rows_cap, N, dtype=torch.int64)
    recv[:, :M] = _stamped(parts, stamp)
    recv_d, res_d = recv.cuda(), res.cuda()
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ep = torch.tensor([epoch], dtype=torch.int32, device="cuda")
    vp = C.c_void_p
    st = qwen3.lib.teeny_tp_gather_add_rms_norm_bf16(vp(recv_d.data_ptr()), rows_cap * N, world, vp(ep.data_ptr()), rnd,
                                                     vp(res_d.data_ptr()), vp(y.data_ptr()), vp(w.cuda().data_ptr()), M, N,
                                                     1e-6, 0, vp(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    total = parts[0].clone()
    for p in range(1, world):             # rank order, f32
        total += parts[p]
    h = res + total.bfloat16()
    assert torch.equal(res_d.cpu(), h)
    assert rel(y, oc.rms_norm_bf16(h, w, 1e-6)) < BF16_TOL


def test_tp_gather_wait_runs_out_and_reports_instead_of_hanging(ops):
    """Partials that never arrive (a peer stopped pushing): with a 2 ms limit the kernel must give up, leave 0x301 in
    the device error word, and the device must keep answering."""
    import ctypes as C
    import time
    from oracle import cpu as oc
    from teenygrad_b200 import qwen3
    world, M, N = 2, 4, 1024
    recv = torch.zeros(world, M, N, dtype=torch.int64, device="cuda")   # stamp 0 everywhere: never this round's
    recv[0] = _stamped(torch.ones(M, N), 1).cuda()                        # rank 0 pushed, rank 1 never does
    res = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(res)
    w = torch.ones(N, dtype=torch.bfloat16, device="cuda")
    ep = torch.zeros(1, dtype=torch.int32, device="cuda")
    vp = C.c_void_p
    t0 = time.time()
    st = qwen3.lib.teeny_tp_gather_add_rms_norm_bf16(vp(recv.data_ptr()), M * N, world, vp(ep.data_ptr()), 0,
                                                     vp(res.data_ptr()), vp(y.data_ptr()), vp(w.data_ptr()), M, N, 1e-6,
                                                     2_000_000, vp(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    assert ops.device_error(clear=True) == 0x301
    assert time.time() - t0 < 1.0, "the bounded wait took far longer than its limit"
    # the context is intact: an ordinary kernel still runs and is right
    x, wt = _gemm_inputs(64, 128, 256)
    assert rel(ops.linear_forward(x.cuda(), wt.cuda()), oc.linear_bf16(x, wt)) < BF16_TOL
    assert ops.device_error(clear=True) == 0


@pytest.mark.parametrize("rows,cols,parts,temperature,top_k,top_p", [
    (8, 151936, 8, 0.8, 50, 0.9), (3, 151936, 2, 1.5, 1024, 0.95), (5, 4096, 4, 0.6, 64, 1.0), (4, 1024, 8, 1.0, 1024, 0.7),
])
def test_sampling_over_vocabulary_shards_equals_the_unsharded_sampler(ops, rows, cols, parts, temperature, top_k, top_p):
    """Per-shard candidate lists + merge (what the vocabulary-parallel LM head does across ranks) must pick exactly the
    token the one-kernel sampler picks on the whole row: same candidates, same order, same sums, same u."""
    import ctypes as C
    g = torch.Generator().manual_seed(rows * 7 + parts)
    logits = (torch.randn(rows, cols, generator=g) * 3).bfloat16()
    logits[0, [1, cols // parts, cols - 1]] = 30.0   # ties across shards: lowest global index first
    u = torch.rand(rows, generator=g)
    want, wprob = ops.sample_top_k_top_p(logits.cuda(), temperature, top_k, top_p, u.cuda(), want_prob=True)
    vl = cols // parts
    lists = torch.zeros(parts, rows, top_k, dtype=torch.int64, device="cuda")
    vp = C.c_void_p
    st = vp(torch.cuda.current_stream().cuda_stream)
    for p in range(parts):
        shard = logits[:, p * vl:(p + 1) * vl].contiguous().cuda()
        rc = ops.lib.teeny_sample_candidates_bf16(vp(shard.data_ptr()), vl, rows, vl, top_k, p * vl, vp(lists[p].data_ptr()), st)
        assert rc == 0
    got = torch.empty(rows, dtype=torch.int32, device="cuda")
    prob = torch.empty(rows, dtype=torch.float32, device="cuda")
    uc = u.cuda()
    rc = ops.lib.teeny_sample_merge(vp(lists.data_ptr()), parts, rows * top_k, rows, temperature, top_k, top_p,
                                    vp(uc.data_ptr()), vp(got.data_ptr()), vp(prob.data_ptr()), st)
    assert rc == 0
    assert torch.equal(got.cpu(), want.cpu())
    assert torch.allclose(prob.cpu(), wprob.cpu(), rtol=1e-6, atol=0)
