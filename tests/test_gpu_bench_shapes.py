"""GPU parity at the shapes the benchmark itself runs (BASELINE configs 2, 3 and 5), through the C ABI.

The CPU oracle cannot redo these sizes in full within a test, so each case runs the GPU at full size and the oracle
on a slice that is independent of the rest by construction: whole sequences of the batch (sequences never interact),
(batch, head) pairs of an attention call, rows of a GEMM.  Bars as everywhere: bf16 within 2e-2 (max|a - e| / max|e|),
token ids equal unless the oracle's own two best logits are a bf16 near-tie.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2


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


# ------------------------------------------------------------------------------------------------ config 2: GEMM
def _gemm_inputs(M, N, K, seed=1):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = ((torch.rand(M, K, generator=g, device="cuda") * 2 - 1) * 0.05).bfloat16()
    w = ((torch.rand(N, K, generator=g, device="cuda") * 2 - 1) * 0.05).bfloat16()
    return x, w


@pytest.mark.parametrize("M,N,K", [
    (4096, 4096, 4096), (4096, 12288, 4096),                   # config 2's large shapes
    (65536, 6144, 4096), (65536, 4096, 4096), (65536, 4096, 12288),  # config 5's prefill projections (32 x 2048 tokens)
])
def test_linear_bf16_full_size_sampled_rows(ops, M, N, K):
    """Full-size launch; the oracle recomputes rows spread over the first, middle and last 256-row tiles."""
    from oracle import cpu as oc
    x, w = _gemm_inputs(M, N, K)
    y = ops.linear_forward(x, w)
    rows = torch.tensor(sorted({0, 1, 127, 128, 255, 256, M // 2 - 1, M // 2, M // 2 + 77, M - 257, M - 256, M - 129,
                                M - 128, M - 2, M - 1}))
    e = oc.linear_bf16(x[rows.cuda()].cpu(), w.cpu())
    assert rel(y[rows.cuda()], e) < TOL
    # the rest of the output through a property: every row's result depends on that row alone, so recomputing a
    # strided subset of rows as a separate (differently tiled) launch must give the same numbers
    sub = torch.arange(0, M, 509, device="cuda")
    y_sub = ops.linear_forward(x[sub].contiguous(), w)
    assert rel(y[sub], y_sub) < 5e-3


def test_linear_swiglu_full_size_sampled_rows(ops):
    """Gate/up projection of config 5's prefill with the SwiGLU epilogue: 65536 x (2 x 12288) x 4096."""
    from oracle import cpu as oc
    M, I, K = 65536, 12288, 4096
    g = torch.Generator(device="cuda").manual_seed(13)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()
    wg = (torch.randn(I, K, generator=g, device="cuda") * 0.02).bfloat16()
    wu = (torch.randn(I, K, generator=g, device="cuda") * 0.02).bfloat16()
    out = ops.linear_swiglu(x, ops.interleave_gate_up(wg, wu))
    rows = torch.tensor([0, 255, 256, 32767, 32768, 65279, 65280, 65535])
    xs = x[rows.cuda()].cpu()
    e = oc.silu_mul_bf16(oc.linear_bf16(xs, wg.cpu()), oc.linear_bf16(xs, wu.cpu()))
    assert rel(out[rows.cuda()], e) < TOL


# ------------------------------------------------------------------------------------------------ config 3: attention
def test_flash_attn_prefill_config3_sampled_heads(ops):
    """Batch 4, 32 query / 8 KV heads, sequence 4096, causal: full launch, oracle on sampled (batch, head) pairs."""
    from oracle import cpu as oc
    B, Hq, Hkv, S, D = 4, 32, 8, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, Hq, S, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, S, D, generator=g, device="cuda").bfloat16()
    o, lse = ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, want_lse=True)
    for (b, h) in [(0, 0), (0, 31), (1, 5), (2, 18), (3, 12), (3, 31)]:
        hk = h // (Hq // Hkv)
        eo, el = oc.attention_bf16(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, hk:hk + 1].cpu(), v[b:b + 1, hk:hk + 1].cpu(),
                                   D ** -0.5, causal=True)
        assert rel(o[b:b + 1, h:h + 1], eo) < TOL, (b, h)
        assert (lse[b:b + 1, h:h + 1].cpu() - el).abs().max() < 2e-2, (b, h)


def test_flash_attn_prefill_bench_shape_sampled_heads(ops):
    """The prefill attention call of config 5: batch 32, sequence 2048, token-major views into the fused projection."""
    from oracle import cpu as oc
    B, Hq, Hkv, S, D = 32, 32, 8, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g, device="cuda").bfloat16()
    q = qkv[:, :Hq * D].view(B, S, Hq, D).permute(0, 2, 1, 3)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D).permute(0, 2, 1, 3)
    v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D).permute(0, 2, 1, 3)
    out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device="cuda")
    ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, out=out.permute(0, 2, 1, 3))
    for (b, h) in [(0, 0), (7, 13), (16, 31), (31, 0), (31, 31)]:
        hk = h // (Hq // Hkv)
        eo, _ = oc.attention_bf16(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, hk:hk + 1].cpu(), v[b:b + 1, hk:hk + 1].cpu(),
                                  D ** -0.5, causal=True)
        assert rel(out.permute(0, 2, 1, 3)[b:b + 1, h:h + 1], eo) < TOL, (b, h)


@pytest.mark.parametrize("B,L", [(32, 2048), (32, 2175), (32, 2304), (4, 4096)])
def test_flash_attn_decode_bench_shapes(ops, B, L):
    """Decode attention as the benchmark launches it on one GPU: batch 32 x 8 KV heads = 256 (sequence, head) pairs,
    which is the kernel's unsplit variant (every CTA walks one whole sequence; smaller launches split the sequence and
    merge), cache capacity 2304 at the first, a middle and the last step's length.  Also config 3's decode variant
    (batch 4, 4096 cached tokens)."""
    from oracle import cpu as oc
    Hq, Hkv, D = 32, 8, 128
    cap = 2304 if B == 32 else 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, Hq, 1, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    eo, _ = oc.attention_bf16(q.cpu(), k[:, :, :L].cpu(), v[:, :, :L].cpu(), D ** -0.5, causal=False)
    k[:, :, L:] = float("nan")  # rows past the live length must never reach the result
    v[:, :, L:] = float("nan")
    o = ops.flash_attn_decode(q, k, v, L, D ** -0.5)
    assert rel(o, eo) < TOL
    o2 = ops.flash_attn_decode(q, k, v, torch.tensor([L], dtype=torch.int32, device="cuda"), D ** -0.5)
    assert torch.equal(o, o2)


# ------------------------------------------------------------------------------------------------ config 5: one layer
def test_qwen3_8b_shaped_layer_full_batch():
    """One decoder layer of the Qwen3-8B shape (hidden 4096, 32 / 8 heads, intermediate 12288, vocabulary 151936,
    untied head) on the benchmark's batch: prefill of 32 x 2048 tokens, then 8 graph-replayed decode steps at batch 32.
    The GPU runs the whole batch; the oracle runs four whole sequences of it.  Checked: the hidden state after the
    layer on all 2048 positions (covers the CTA-pair GEMMs at M = 65536 incl. K = 12288 and the SwiGLU epilogue, the
    prefill RoPE / cache kernel and prefill attention at batch 32), then per decode step the logits (decode attention
    with its fused head norm / RoPE / cache append at 256 (sequence, head) pairs, the cluster split-K GEMMs, the LM
    head) with the oracle fed the GPU's tokens, and the GPU's pick against the oracle's argmax."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import qwen3 as oq
    from teenygrad_b200 import qwen3
    B, S, steps, H = 32, 2048, 9, 4096
    cfg = qwen3.Qwen3Config(1, H, 32, 8, 128, 12288, 151936, tied=False)
    r = qwen3.Qwen3Runner(cfg, max_batch=B, max_len=S + steps, max_tokens=B * S, max_new_tokens=steps)
    sd = dict(qwen3.random_weights_device(cfg, 4, r.device))
    r.load_state_dict(sd)
    ids = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(4))
    pick = [0, 9, 22, 31]
    ocfg = oq.OracleQwen3Config(1, H, 32, 8, 128, 12288, 151936, tied=False)
    oracle = oq.OracleQwen3(ocfg, {k: v.cpu() for k, v in sd.items()})
    del sd

    r.prefill(ids)
    residual, delta = r.residual_stream(B * S)
    got_hidden = (residual.view(B, S, H)[pick, :S - 1] + delta.view(B, S, H)[pick, :S - 1]).cpu()
    got_last = residual.view(B, S, H)[pick, S - 1].cpu()  # the head already added the last position's delta in place
    got_logits = r.logits()[pick].cpu()
    got_ids = r.next_ids()[pick].cpu().long()

    want_logits = oracle.forward(ids[pick].long())
    want_hidden = oracle.last_residual
    assert rel(got_hidden, want_hidden[:, :S - 1]) < TOL
    assert rel(got_last, want_hidden[:, S - 1]) < TOL
    scale = float(want_logits.float().abs().max())

    def check_step(t, got_logits, got_ids, want_logits):
        err = float((got_logits.float() - want_logits.float()).abs().max()) / scale
        assert err < TOL, f"step {t}: logits differ from the oracle by {err}"
        want_ids = torch.argmax(want_logits.float(), dim=-1)
        for i in range(len(pick)):
            if got_ids[i] != want_ids[i]:  # only acceptable where the oracle's own best two are a bf16 near-tie
                gap = float(want_logits[i].float().max() - want_logits[i, got_ids[i]].float()) / scale
                assert gap < TOL, f"step {t} sequence {pick[i]}: picked a token {gap} below the oracle's best"

    check_step(0, got_logits, got_ids, want_logits)
    for t in range(1, steps):
        r.decode_step(graph=True)
        want_logits = oracle.forward(got_ids[:, None])  # the oracle follows the GPU's tokens
        got_logits, got_ids = r.logits()[pick].cpu(), r.next_ids()[pick].cpu().long()
        check_step(t, got_logits, got_ids, want_logits)
    assert qwen3.lib.teeny_device_error(1) == 0
