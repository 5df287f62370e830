"""Kernel micro-benchmarks and profiler cases for libteeny_b200.so.

    python -m teenygrad_b200.microbench time [gemm] [skinny] [prefill] [decode] [elementwise] [sampling]   # CUDA-event timings
    python -m teenygrad_b200.microbench case gemm|skinny|prefill|decode           # a few launches of one kernel
    python -m teenygrad_b200.microbench layers [N]                                # N-layer Qwen3-8B-shaped prefill + 3 decode steps
    python -m teenygrad_b200.microbench trace [N [first [count [shard]]]]         # timeline of one graph-replayed decode step
    python -m teenygrad_b200.microbench tracecase gemm|skinny|prefill|decode      # phase counters of one kernel
    python -m teenygrad_b200.microbench timeline                                  # event order inside one CTA pair of the prefill attention kernel
    python -m teenygrad_b200.microbench probe                                     # tcgen05.mma issue rate from one / two threads

``time`` prints achieved TFLOP/s or GB/s next to cuBLAS / cuDNN (torch) on the same inputs.  Large kernels are timed
one launch at a time with an L2 flush (a 256 MB write) before each; the decode-shaped kernels, which last tens of
microseconds, are captured in a CUDA graph over rotating copies of their inputs (larger than L2 together) so neither
host launch overhead nor a warm L2 enters the number.  ``case`` and ``layers`` exist to be run under ``ncu``.
``trace``, ``tracecase``, ``timeline`` and ``probe`` need a library with per-CTA timer records: ``make -C teenygrad_b200/csrc OBJDIR=_obj_trace
OUT=../libteeny_b200_trace.so EXTRA=-DTEENY_TRACE`` and ``TEENY_B200_LIB=teenygrad_b200/libteeny_b200_trace.so``.
"""
import sys

import torch

from . import ops

HQ, HKV, D = 32, 8, 128


def _graph_time(fns, reps=5):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
    return a.elapsed_time(b) / reps / len(fns)


_flush = None


def _flushed_time(fn, iters=8, warm=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def _rand(*shape):
    return (torch.rand(*shape, device="cuda") * 0.1 - 0.05).bfloat16()


def time_gemm():
    for (M, N, K) in [(4096, 4096, 4096), (4096, 12288, 4096), (8192, 8192, 8192), (65536, 6144, 4096), (65536, 4096, 12288)]:
        x, w = _rand(M, K), _rand(N, K)
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        t = _flushed_time(lambda: ops.linear_forward(x, w, out=y))
        t2 = _flushed_time(lambda: torch.matmul(x, w.t(), out=y))
        fl = 2 * M * N * K
        print(f"linear bf16 {M}x{N}x{K}: {t:.4f} ms {fl / t / 1e9:.0f} TFLOP/s | cuBLAS {t2:.4f} ms {fl / t2 / 1e9:.0f} TFLOP/s", flush=True)


def time_skinny():
    for (M, N, K) in [(32, 24576, 4096), (32, 4096, 12288), (32, 6144, 4096), (32, 4096, 4096), (1, 4096, 4096),
                      (128, 4096, 4096), (32, 151936, 4096)]:
        n = max(2, int(1.5e9 // (N * K * 2)))
        ws = [_rand(N, K) for _ in range(n)]
        x = _rand(M, K)
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        t = _graph_time([(lambda w=w: ops.linear_forward(x, w, out=y)) for w in ws])
        t2 = _graph_time([(lambda w=w: torch.matmul(x, w.t(), out=y)) for w in ws])
        by = 2 * (M * K + N * K + M * N)
        print(f"linear bf16 {M}x{N}x{K}: {t * 1e3:.1f} us {by / t / 1e6:.0f} GB/s | cuBLAS {t2 * 1e3:.1f} us {by / t2 / 1e6:.0f} GB/s", flush=True)


def time_w8():
    """The decode GEMM shapes with bf16 weights and with FP8 (E4M3, per-channel scales) weights."""
    from . import quant
    for (M, N, K, swiglu) in [(32, 6144, 4096, False), (32, 4096, 4096, False), (32, 24576, 4096, True), (32, 4096, 12288, False),
                              (32, 151936, 4096, False), (1, 4096, 4096, False), (128, 4096, 4096, False)]:
        n = max(2, int(300e6 // (N * K)) + 1)
        ws = [_rand(N, K) for _ in range(n)]
        qs = [quant.quantize_fp8(w) for w in ws]
        x = _rand(M, K)
        y = torch.empty(M, N // 2 if swiglu else N, dtype=torch.bfloat16, device="cuda")
        f16 = [(lambda w=w: (ops.linear_swiglu if swiglu else ops.linear_forward)(x, w, out=y)) for w in ws]
        f8 = [(lambda q=q: ops.linear_w8a16(x, q.q, q.scale, "channel", out=y, swiglu=swiglu)) for q in qs]
        x8, xs = ops.split_fp8(x)
        f88 = [(lambda q=q: ops.linear_w8a8x2(x8, xs, q.q, q.scale, "channel", out=y, swiglu=swiglu)) for q in qs]
        t16, t8, t88 = _graph_time(f16), _graph_time(f8), _graph_time(f88)
        print(f"linear {M}x{N}x{K}{' + SwiGLU' if swiglu else ''}: bf16 weights {t16 * 1e3:.1f} us ({N * K * 2 / t16 / 1e6:.0f} GB/s)"
              f" | FP8 weights {t8 * 1e3:.1f} us ({N * K / t8 / 1e6:.0f} GB/s)"
              f" | FP8 weights, two-term FP8 activations {t88 * 1e3:.1f} us ({N * K / t88 / 1e6:.0f} GB/s)", flush=True)


def time_prefill():
    for (B, S) in [(4, 4096), (32, 2048)]:
        q = torch.randn(B, HQ, S, D, device="cuda").bfloat16()
        k = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
        v = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        t = _flushed_time(lambda: ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, out=o))
        t2 = _flushed_time(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True))
        fl = 0.5 * 4 * B * HQ * S * S * D
        print(f"flash-attn causal B{B} S{S}: {t:.3f} ms {fl / t / 1e9:.0f} TFLOP/s | torch SDPA {t2:.3f} ms {fl / t2 / 1e9:.0f} TFLOP/s", flush=True)


def time_decode():
    for (B, L) in [(32, 2304), (32, 2048), (4, 4096)]:
        n = max(2, int(1.2e9 // (2 * B * HKV * L * D * 2)))
        q = torch.randn(B, HQ, 1, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        kv = [(torch.randn(B, HKV, L, D, device="cuda").bfloat16(), torch.randn(B, HKV, L, D, device="cuda").bfloat16())
              for _ in range(n)]
        sc = torch.empty(ops.lib.teeny_attn_decode_scratch_bytes(B, HQ, D, L), dtype=torch.uint8, device="cuda")
        t = _graph_time([(lambda k=k, v=v: ops.flash_attn_decode(q, k, v, L, D ** -0.5, out=o, scratch=sc)) for k, v in kv])
        by = 2 * B * HKV * L * D * 2
        print(f"flash-attn decode B{B} L{L}: {t * 1e3:.1f} us {by / t / 1e6:.0f} GB/s", flush=True)


def time_elementwise():
    """The two bandwidth-bound prefill passes at the bench's size (32 x 2048 tokens of Qwen3-8B)."""
    T, S, H = 65536, 2048, 4096
    qkv = _rand(T, (HQ + 2 * HKV) * D)
    qw, kw = torch.ones(D, device="cuda").bfloat16(), torch.ones(D, device="cuda").bfloat16()
    inv = (1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)).cuda()
    cos, sin = ops.rope_table(inv, S)
    kc = torch.empty(T // S, HKV, S, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.empty_like(kc)
    t = _flushed_time(lambda: ops.qk_norm_rope_kv(qkv, qw, kw, cos, sin, kc, vc, S, HQ, HKV, 0, 1e-6))
    by = 2 * (qkv.numel() + T * HQ * D + 2 * kc.numel())
    print(f"qk_norm_rope_kv {T} tokens: {t * 1e3:.0f} us {by / t / 1e6:.0f} GB/s", flush=True)
    x, res, w = _rand(T, H), _rand(T, H), torch.ones(H, device="cuda").bfloat16()
    t = _flushed_time(lambda: ops.add_rms_norm(x, res, w, 1e-6))
    by = 2 * 4 * x.numel()
    print(f"add_rms_norm {T}x{H}: {t * 1e3:.0f} us {by / t / 1e6:.0f} GB/s (includes the output allocation)", flush=True)


def time_sampling():
    logits = (torch.randn(32, 151936, device="cuda") * 3).bfloat16()
    u = torch.rand(32, device="cuda")
    for k in (50, 1024):
        t = _flushed_time(lambda: ops.sample_top_k_top_p(logits, 0.8, k, 0.9, u))
        print(f"sample_top_k_top_p 32 x 151936, top_k {k}: {t * 1e3:.0f} us (three passes over 9.7 MB of logits)", flush=True)


def case(which):
    """A handful of launches of one kernel on inputs larger than L2 (for ncu -k ... -s 2 -c 2)."""
    if which == "gemm":
        M, N, K = 4096, 12288, 4096
        x, w = _rand(M, K), _rand(N, K)
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for _ in range(4):
            ops.linear_forward(x, w, out=y)
    elif which == "skinny":
        M, N, K = 32, 6144, 4096
        x, ws = _rand(M, K), [_rand(N, K) for _ in range(4)]
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        for w in ws:
            ops.linear_forward(x, w, out=y)
    elif which == "w8":  # the gate/up projection of the decode step with FP8 weights
        from . import quant
        M, N, K = 32, 24576, 4096
        x = _rand(M, K)
        qs = [quant.quantize_fp8(_rand(N, K)) for _ in range(3)]
        y = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
        for q in qs:
            ops.linear_w8a16(x, q.q, q.scale, "channel", out=y, swiglu=True)
    elif which == "prefill":
        B, S = 4, 4096
        q = torch.randn(B, HQ, S, D, device="cuda").bfloat16()
        k = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
        v = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        for _ in range(3):
            ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, out=o)
    elif which == "decode":
        B, L = 32, 2304
        q = torch.randn(B, HQ, 1, D, device="cuda").bfloat16()
        k = torch.randn(B, HKV, L, D, device="cuda").bfloat16()
        v = torch.randn(B, HKV, L, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        for _ in range(4):
            ops.flash_attn_decode(q, k, v, L, D ** -0.5, out=o)
    else:
        raise SystemExit(f"unknown case {which}")
    torch.cuda.synchronize()


def layers(n_layers):
    """Prefill (batch 32 x 2048) and three eager decode steps of an n-layer Qwen3-8B-shaped model: every kernel of the
    runner at its full per-launch size, few enough launches for a profiler launch list."""
    from . import qwen3
    cfg = qwen3.Qwen3Config(n_layers, 4096, 32, 8, 128, 12288, 151936, tied=False)
    r = qwen3.Qwen3Runner(cfg, max_batch=32, max_len=2304, max_tokens=32 * 2048, max_new_tokens=8)
    qwen3.load_random_weights(r, 4)
    ids = torch.randint(0, cfg.vocab, (32, 2048), dtype=torch.int32)
    r.prefill(ids)
    for _ in range(3):
        r.decode_step(graph=False)
    torch.cuda.synchronize()


def trace(n_layers, first=0, count=48, shard=1):
    """Prints, for every kernel launch of one graph-replayed decode step (batch 32, cache length ~2050) of an
    n-layer Qwen3-8B-shaped model: CTAs, first/last CTA resident, first/last CTA released by its dependency wait,
    first/last CTA finished (where the kernel records it), in microseconds from the start of the step.  Prints
    ``count`` launches starting at launch number ``first`` (under tensor parallelism the first layer absorbs the
    ranks' start skew, so look further in).  ``shard`` > 1 on one GPU runs one rank's shard of a ``shard``-way
    tensor-parallel split (heads, intermediate and vocabulary divided, no exchange): the per-layer time a rank would
    have if the cross-rank reductions were free."""
    import ctypes
    from collections import defaultdict

    import numpy as np

    from . import qwen3
    lib = ops.lib
    if not hasattr(lib, "teeny_trace_count"):
        raise SystemExit("library was built without -DTEENY_TRACE")
    lib.teeny_trace_name.restype = ctypes.c_char_p
    lib.teeny_trace_name.argtypes = [ctypes.c_int]
    lib.teeny_trace_dump.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint, ctypes.c_int]

    def dump():
        ev = []
        for i in range(lib.teeny_trace_count()):
            name = lib.teeny_trace_name(i).decode().split("/")[-1]
            buf = np.zeros((1 << 18, 4), dtype=np.uint64)
            n = lib.teeny_trace_dump(i, buf.ctypes.data, 1 << 18, 1)
            for r in buf[:n]:
                ev.append((name, int(r[2]) & 0xFFFFFFFF, int(r[0]), int(r[1]), int(r[3]) >> 32))
        return ev

    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    comm = None
    if world > 1:  # tensor parallel: launched by torch.distributed.run, rank 0 prints its own timeline
        import torch.distributed as dist

        from . import tp
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        comm = tp.init_comm(rank, world)
    cfg = qwen3.Qwen3Config(n_layers, 4096, 32 // shard, 8 // shard, 128, 12288 // shard, 151936 // shard, tied=False)
    r = qwen3.Qwen3Runner(cfg, max_batch=32, max_len=2304, max_tokens=32 * 2048, max_new_tokens=16,
                          tp_rank=rank, tp_size=world, comm=comm)
    qwen3.load_random_weights(r, 4)
    r.prefill(torch.randint(0, cfg.vocab, (32, 2048), dtype=torch.int32, generator=torch.Generator().manual_seed(5)))
    for _ in range(4):
        r.decode_step(graph=True)
    torch.cuda.synchronize()
    dump()
    r.decode_step(graph=True)
    torch.cuda.synchronize()
    ev = dump()
    if world > 1:
        dist.barrier()
    if rank != 0:
        return
    waits = sorted((e for e in ev if e[2] > 15), key=lambda e: e[2])
    ends, marks = defaultdict(list), defaultdict(list)
    for e in ev:
        if e[2] == 0:
            ends[(e[0], e[4])].append(e[3])
        elif e[2] <= 15:
            marks[(e[0], e[4], e[2])].append(e[3])
    t0 = waits[0][2]
    launches = defaultdict(list)  # (file, line, grid) -> list of launches, each a list of records
    for e in waits:
        ls = launches[(e[0], e[1], e[4])]
        if ls and len(ls[-1]) < e[4] and e[2] - ls[-1][0][2] < 300000:
            ls[-1].append(e)
        else:
            ls.append([e])
    flat = sorted(((k, l) for k, ls in launches.items() for l in ls), key=lambda kl: min(e[3] for e in kl[1]))
    print(f"{'kernel (file:line of its wait)':34s} {'ctas':>5s} {'in0':>8s} {'inN':>8s} {'go0':>8s} {'goN':>8s} {'end0':>8s} {'endN':>8s}")
    for (name, line, grid), l in flat[first:first + count]:
        us = lambda t: (t - t0) / 1e3
        go0 = min(e[3] for e in l)
        es = sorted(t for t in ends.get((name, grid), []) if go0 <= t < go0 + 300000)[:grid]
        print(f"{name[:26] + ':' + str(line):34s} {len(l):5d} {us(min(e[2] for e in l)):8.1f} {us(max(e[2] for e in l)):8.1f} "
              f"{us(go0):8.1f} {us(max(e[3] for e in l)):8.1f} "
              f"{us(es[0]) if es else float('nan'):8.1f} {us(es[-1]) if es else float('nan'):8.1f}", end="")
        for mid in range(1, 16):  # intermediate marks: median over the launch's CTAs
            ms = sorted(t for t in marks.get((name, grid, mid), []) if go0 <= t < go0 + 300000)[:grid]
            if ms:
                print(f"  m{mid}={us(ms[len(ms) // 2]):.1f}", end="")
        print()


def tracecase(which):
    """Runs ``case`` and prints, per source line and id, count / mean / sum of the TRACE_VALUE records (and the mean
    dependency-wait interval per kernel).  Needs a -DTEENY_TRACE build."""
    import ctypes
    from collections import defaultdict

    import numpy as np
    lib = ops.lib
    if not hasattr(lib, "teeny_trace_count"):
        raise SystemExit("library was built without -DTEENY_TRACE")
    lib.teeny_trace_name.restype = ctypes.c_char_p
    lib.teeny_trace_name.argtypes = [ctypes.c_int]
    lib.teeny_trace_dump.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint, ctypes.c_int]
    case(which)
    acc = defaultdict(list)
    for i in range(lib.teeny_trace_count()):
        name = lib.teeny_trace_name(i).decode().split("/")[-1]
        buf = np.zeros((1 << 18, 4), dtype=np.uint64)
        n = lib.teeny_trace_dump(i, buf.ctypes.data, 1 << 18, 1)
        b = buf[:n]
        for r in b[(b[:, 0] >= 16) & (b[:, 0] < 32)]:
            if int(r[1]) >> 40:  # a clock stamp of ``timeline``, not a counter
                continue
            acc[(name, int(r[2]) & 0xFFFFFFFF, int(r[0]) - 16)].append(int(r[1]))
    for (name, line, vid), vals in sorted(acc.items()):
        print(f"{name}:{line} value {vid:2d}: n {len(vals):6d} mean {sum(vals) / len(vals):12.1f} sum {sum(vals):14d}")


def timeline():
    """Prints, in order, the clock stamps the prefill attention kernel keeps for twenty key tiles of its first CTA pair
    (S buffer free / Q K^T issued / S arrived / row loaded / maximum decided / exponentials done / P buffer free /
    P stored / P V issued / item closed or next item opened): the steady state of the pair and one item boundary.
    Needs a -DTEENY_TRACE build."""
    import ctypes

    import numpy as np
    lib = ops.lib
    if not hasattr(lib, "teeny_trace_count"):
        raise SystemExit("library was built without -DTEENY_TRACE")
    lib.teeny_trace_name.restype = ctypes.c_char_p
    lib.teeny_trace_name.argtypes = [ctypes.c_int]
    lib.teeny_trace_dump.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint, ctypes.c_int]
    names = {0: "QK issuer: S buffer free", 1: "QK issuer: issued", 2: "PV issuer: P full", 9: "PV issuer: issued",
             3: "softmax: S arrived", 4: "softmax: row loaded, maximum", 5: "softmax: maximum decided",
             6: "softmax: exponentials done", 7: "softmax: P buffer free", 8: "softmax: P stored",
             10: "softmax: item closed (output on its way)", 11: "softmax: next item opened (Q in tensor memory)"}
    B, S = 4, 4096
    q = torch.randn(B, HQ, S, D, device="cuda").bfloat16()
    k = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
    v = torch.randn(B, HKV, S, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    recs = []
    for _ in range(3):  # the last launch is the one printed
        ops.flash_attn_fwd(q, k, v, D ** -0.5, causal=True, out=o)
        torch.cuda.synchronize()
        recs = []
        for i in range(lib.teeny_trace_count()):
            buf = np.zeros((1 << 18, 4), dtype=np.uint64)
            n = lib.teeny_trace_dump(i, buf.ctypes.data, 1 << 18, 1)
            if b"attention_prefill" not in lib.teeny_trace_name(i):
                continue
            for r in buf[:n][(buf[:n, 0] >= 16) & (buf[:n, 0] < 32)]:
                val = int(r[1])
                if val >> 40:  # (key tile << 40) | clock
                    recs.append((val & ((1 << 40) - 1), val >> 40, int(r[0]) - 16))
    recs.sort()
    print("cycles  key tile  group  event   (causal, batch 4, 32 / 8 heads, sequence 4096; CTA pair 0)")
    for t, g, i in recs:
        print(f"{t - recs[0][0]:7d}  {g:4d}  {'AB'[g & 1]}  {names.get(i, i)}")


def probe():
    """Cycles per tcgen05.mma when one thread (or two, in different warps) issues 4096 of them from a loop: the
    figures behind the attention kernel's straight-line issue blocks and its two issuer threads.  Needs a
    -DTEENY_TRACE build."""
    import ctypes
    lib = ops.lib
    if not hasattr(lib, "teeny_probe_mma_issue"):
        raise SystemExit("library was built without -DTEENY_TRACE")
    iters = 4096
    print("cta_group  M    N    A operand   issuers / accumulators   cycles per MMA (issue, completed)   pipe needs")
    for pair, n, mode in [(0, 128, 0), (0, 128, 1), (0, 128, 2), (0, 128, 5), (0, 64, 1), (0, 256, 0), (0, 256, 1),
                          (1, 128, 0), (1, 128, 1), (1, 128, 5), (1, 128, 4), (1, 256, 0), (1, 256, 4)]:
        out = (ctypes.c_longlong * 2)()
        rc = lib.teeny_probe_mma_issue(pair, mode, n, iters, out)
        if rc != 0:
            raise SystemExit(f"probe failed: {rc}")
        m = 256 if pair else 128
        need = m * n * 16 * 2 / 8192 / (2 if pair else 1)
        who = "two threads" if mode & 4 else ("one thread, two accumulators" if mode & 2 else "one thread")
        print(f"{'::2' if pair else '::1':9s} {m:4d} {n:4d}  {'tensor mem' if mode & 1 else 'shared mem':10s}  {who:28s} "
              f"{out[0] / iters:7.1f} {out[1] / iters:7.1f}   {need:5.0f}")


def main(argv):
    import os
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    mode = argv[0] if argv else "time"
    if mode == "time":
        what = argv[1:] or ["gemm", "skinny", "prefill", "decode", "elementwise", "sampling"]
        for name in what:
            {"gemm": time_gemm, "skinny": time_skinny, "prefill": time_prefill, "decode": time_decode,
             "elementwise": time_elementwise, "sampling": time_sampling, "w8": time_w8}[name]()
    elif mode == "case":
        case(argv[1])
    elif mode == "probe":
        probe()
    elif mode == "tracecase":
        tracecase(argv[1])
    elif mode == "timeline":
        timeline()
    elif mode == "layers":
        layers(int(argv[1]) if len(argv) > 1 else 6)
    elif mode == "trace":
        trace(*(int(v) for v in argv[1:5])) if len(argv) > 1 else trace(8)
    else:
        raise SystemExit(__doc__)
    print("device error word:", ops.device_error())


if __name__ == "__main__":
    main(sys.argv[1:])
