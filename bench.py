#!/usr/bin/env python
"""Headline benchmark: Qwen3-8B-shaped greedy generation (batch 32, prefill 2048, 256 new tokens), bf16,
tensor-parallel over N GPUs of one node; value = tokens (prompt + generated) per second over the whole job.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU arm: the Qwen3 forward the reference runs (PyTorch CPU)

A "step" is one full generation: prefill of 32 x 2048 prompt tokens, then 255 CUDA-graph decode steps (the first
new token comes out of the prefill).  Weights are seeded random-init tensors of the Qwen3-8B shapes and prompts are
uniform random ids (no checkpoints or datasets on this machine): `data` says synthetic.

One JSON line on stdout (rank 0).  `value` is timed with CUDA events with everything already on the device; `e2e`
is the same job through the public API (`Qwen3Runner.generate`) with the prompt ids in pinned host memory and the
generated ids copied back, host<->device copies inside the timed region.  `roofline` is for the dominant kernel,
the tcgen05 GEMM, timed live on this run's four prefill GEMM shapes.  `cpu_baseline` is the CPU port of the path
(oracle/qwen3.py, PyTorch CPU threads) timed on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

_JSON_OUT = None  # duplicate of the original stdout, opened in main()

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "qwen3_8b_tokens_per_s"
UNIT = "tok/s"
# bounded CPU sample of the workload (sized for roughly 10-30 s of host work on a 16-thread box)
CPU_SAMPLE = dict(sample_layers=4, batch=16, prefill=2048, new_tokens=16)
# per-step sample of the --impl reference arm: a quarter of that, so warm-up + steps stay within a few minutes
REF_SAMPLE = dict(sample_layers=2, batch=8, prefill=2048, new_tokens=8)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # workload knobs (defaults = BASELINE config 5); smaller values are for debugging only and are echoed in `config`
    p.add_argument("--layers", type=int, default=36)
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--prefill", type=int, default=2048)
    p.add_argument("--new-tokens", type=int, default=256)
    p.add_argument("--no-cpu-baseline", action="store_true")
    return p.parse_args()


# ------------------------------------------------------------------------------------------------ peaks / clocks
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        time.sleep(0.05)
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        smax = next((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), None)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": smax, "reasons": reasons,
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_generation_rate(cfg_kwargs, sample_layers, batch, prefill, new_tokens, threads=None):
    """Times the CPU port of the path (oracle.qwen3.OracleQwen3 -- the op sequence HF transformers runs for the
    reference's Qwen3 script, on PyTorch CPU) on `sample_layers` layers of the real shapes and scales the layer time
    to the full depth.  Returns (tok/s for the full-depth model on the sample's batch/prompt, description)."""
    import torch
    from oracle import qwen3 as oq
    if threads:
        torch.set_num_threads(threads)
    full_layers = cfg_kwargs["num_layers"]
    kw = dict(cfg_kwargs)
    kw["num_layers"] = sample_layers
    cfg = oq.OracleQwen3Config(**kw)
    # timing does not depend on the values: every tensor is a view into one random block (fast to create)
    H, D = cfg.hidden, cfg.head_dim
    biggest = max(cfg.vocab * H, cfg.intermediate * H)
    block = (torch.randn(biggest // 64 + 1, generator=torch.Generator().manual_seed(4)) * 0.02).bfloat16().repeat(64)

    def view(*shape):
        n = 1
        for s in shape:
            n *= s
        return block[:n].view(*shape)

    sd = {"model.embed_tokens.weight": view(cfg.vocab, H), "model.norm.weight": torch.ones(H, dtype=torch.bfloat16)}
    if not cfg.tied:
        sd["lm_head.weight"] = view(cfg.vocab, H)
    for i in range(sample_layers):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = view(cfg.num_q_heads * D, H)
        sd[p + "self_attn.k_proj.weight"] = view(cfg.num_kv_heads * D, H)
        sd[p + "self_attn.v_proj.weight"] = view(cfg.num_kv_heads * D, H)
        sd[p + "self_attn.o_proj.weight"] = view(H, cfg.num_q_heads * D)
        sd[p + "mlp.gate_proj.weight"] = view(cfg.intermediate, H)
        sd[p + "mlp.up_proj.weight"] = view(cfg.intermediate, H)
        sd[p + "mlp.down_proj.weight"] = view(H, cfg.intermediate)
        for n in ("self_attn.q_norm.weight", "self_attn.k_norm.weight"):
            sd[p + n] = torch.ones(D, dtype=torch.bfloat16)
        for n in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            sd[p + n] = torch.ones(H, dtype=torch.bfloat16)
    ids = torch.randint(0, cfg.vocab, (batch, prefill), generator=torch.Generator().manual_seed(5))

    def run(layers_cfg):
        m = oq.OracleQwen3(layers_cfg, sd)
        t0 = time.perf_counter()
        m.generate(ids, new_tokens)
        return time.perf_counter() - t0

    zero = oq.OracleQwen3Config(**{**kw, "num_layers": 0})
    run(zero)                      # warm-up of the head path (thread pools, allocator)
    t_head = run(zero)             # embedding + final norm + LM head + argmax only
    t_some = run(cfg)
    per_layer = max(t_some - t_head, 0.0) / sample_layers
    t_full = t_head + per_layer * full_layers
    tokens = batch * (prefill + new_tokens)
    desc = (f"{sample_layers} of {full_layers} layers + embedding/LM head timed, layer time scaled to {full_layers}; "
            f"batch {batch}, prefill {prefill}, {new_tokens} greedy tokens; PyTorch CPU bf16, "
            f"{torch.get_num_threads()} threads; measured {t_some:.2f}s (+{t_head:.2f}s head-only)")
    return tokens / t_full, desc, torch.get_num_threads()


def reference_arm(args, cfg_kwargs):
    """The reference's CPU execution of the path (its Qwen3 script runs the traced PyTorch graph on the CPU,
    support/teeny-torch/python/teenygrad/atlas/module.py:42-45).  The Rust crates cannot be built here (no cargo,
    no teenyc), so this times the CPU port of that op sequence on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    desc, threads = "", 1
    for i in range(args.warmup + args.steps):
        v, desc, threads = cpu_generation_rate(cfg_kwargs, **REF_SAMPLE)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    tokens = REF_SAMPLE['batch'] * (REF_SAMPLE['prefill'] + REF_SAMPLE['new_tokens'])
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * tokens / value,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), file=_JSON_OUT or sys.stdout, flush=True)


def workload_config(args, n):
    return {"workload": f"Qwen3-8B-shaped decoder ({args.layers} layers, hidden 4096, 32 q / 8 kv heads, head_dim 128, "
                        f"intermediate 12288, vocab 151936, untied head), random-init bf16 seed 4; batch {args.batch}, "
                        f"prefill {args.prefill} uniform-random ids, {args.new_tokens} greedy tokens",
            "global_batch": args.batch, "seq_len": args.prefill, "new_tokens": args.new_tokens,
            "parallelism": f"tp{n}", "l2": "inputs larger than L2 (16 GB of weights + KV cache stream every step)"}


# ------------------------------------------------------------------------------------------------ GPU arm
def main():
    args = parse_args()
    # Keep stdout to the one JSON line: libraries write there at the file-descriptor level (NCCL prints its version
    # banner to fd 1 at NCCL_DEBUG=VERSION and WARN), so fd 1 is pointed at stderr for the whole run and the line goes
    # to a private duplicate of the original stdout.
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    cfg_kwargs = dict(num_layers=args.layers, hidden=4096, num_q_heads=32, num_kv_heads=8, head_dim=128,
                      intermediate=12288, vocab=151936, eps=1e-6, rope_theta=1e6, tied=False)
    if args.impl == "reference":
        reference_arm(args, cfg_kwargs)
        return

    import torch
    import torch.distributed as dist
    from teenygrad_b200 import ops, qwen3, tp
    from teenygrad_b200._lib import lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = tp.init_comm(rank, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    B, S, NEW = args.batch, args.prefill, args.new_tokens
    cfg = qwen3.Qwen3Config(**cfg_kwargs)
    runner = qwen3.Qwen3Runner(cfg, max_batch=B, max_len=S + NEW, max_tokens=B * S, max_new_tokens=NEW,
                               tp_rank=rank, tp_size=world, comm=comm)
    qwen3.load_random_weights(runner, seed=4)
    tp_mode = "none" if world == 1 else ("peer-push" if lib.teeny_tp_peer_enabled(comm) else "nccl-allreduce")
    g = torch.Generator().manual_seed(4)
    prompts_host = torch.randint(0, cfg.vocab, (B, S), generator=g, dtype=torch.int32).pin_memory()
    prompts_dev = prompts_host.to(dev)
    out_host = torch.empty(B, NEW, dtype=torch.int32).pin_memory()
    tokens_per_step = B * (S + NEW)

    def one_generation_device():
        return runner.generate(prompts_dev, NEW, use_graph=True)

    def one_generation_e2e():
        ids = prompts_host.to(dev, non_blocking=True)         # H2D of this step's inputs
        out = runner.generate(ids, NEW, use_graph=True)
        out_host.copy_(out, non_blocking=True)                # D2H of the step's result
        torch.cuda.current_stream().synchronize()

    for _ in range(max(args.warmup, 3)):
        one_generation_device()
    barrier()

    # ---- timed region: device-resident inputs ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pre = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    e0.record()
    for i in range(args.steps):
        pre[i][0].record()
        runner.prefill(prompts_dev)
        pre[i][1].record()
        for _ in range(NEW - 1):
            runner.decode_step(graph=True)
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1), sum(a.elapsed_time(b) for a, b in pre)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms, prefill_ms = float(ms[0]), float(ms[1])
    err = lib.teeny_device_error(1)
    if err != 0:
        raise SystemExit(f"device error word {err:#x} after the timed region")

    # ---- end to end through the public API, host buffers ----
    one_generation_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_generation_e2e()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)

    # ---- dominant kernel: the tcgen05 GEMM on this run's prefill shapes (per rank), CUDA events ----
    peaks = measured_peaks()
    T = B * S
    shapes = [(T, (32 + 16) * 128 // world, 4096), (T, 4096, 4096 // world),
              (T, 2 * 12288 // world, 4096), (T, 4096, 12288 // world)]
    flops = gemm_ms = gemm_bytes = 0.0
    x = torch.empty(T, 12288, dtype=torch.bfloat16, device=dev).normal_(0, 0.05)
    wbuf = torch.empty(2 * 12288 * 4096 // world + 4096 * 6144, dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
    ybuf = torch.empty(T * max(2 * 12288 // world, 4096 + 2048), dtype=torch.bfloat16, device=dev)
    for (m, n, k) in shapes:
        xv, wv, yv = x[:, :k], wbuf[:n * k].view(n, k), ybuf[:m * n].view(m, n)
        for _ in range(2):
            ops.linear_forward(xv, wv, out=yv)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            ops.linear_forward(xv, wv, out=yv)
        b.record()
        torch.cuda.synchronize()
        gemm_ms += a.elapsed_time(b) / 3
        flops += 2.0 * m * n * k
        gemm_bytes += 2.0 * (m * k + n * k + m * n)
    achieved = flops / (gemm_ms * 1e-3) / 1e12
    del x, wbuf, ybuf

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    steps = args.steps
    ov = os.environ.get("TEENY_TP_OVERLAP")  # the library's default: overlapped from 8 ranks on
    prefill_overlap = world > 1 and ((ov == "1") if ov else world >= 8)
    value = tokens_per_step * steps / (total_ms * 1e-3)
    decode_ms = total_ms - prefill_ms
    L = cfg.num_layers
    # this library's kernels only (NCCL's are not counted).  Prefill: embedding; per layer norm, QKV GEMM,
    # norm+RoPE+cache, attention, O GEMM, add+norm, gate/up GEMM with SwiGLU epilogue, down GEMM; final add+norm, LM head,
    # argmax (+ merge when tp > 1), generation-state kernels.  Decode: the attention kernel also does the head norms,
    # RoPE, cache append and the merge of split sequences, so a layer is seven launches.
    launches_prefill = 1 + L * 8 + 3 + 2 + (1 if world > 1 else 0)
    launches_decode = 1 + L * 7 + 3 + 1 + (1 if world > 1 else 0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {**workload_config(args, world), "tp_decode_reduction": tp_mode, "tp_prefill_reduction":
                   "none" if world == 1 else ("nccl-allreduce, overlapped with the other half-batch's compute"
                                              if prefill_overlap else "nccl-allreduce")},
        "phases": {"prefill_ms": prefill_ms / steps, "decode_ms": decode_ms / steps,
                   "prefill_tok_s": B * S * steps / (prefill_ms * 1e-3),
                   "decode_tok_s": B * (NEW - 1) * steps / (decode_ms * 1e-3),
                   "decode_ms_per_token_step": decode_ms / steps / (NEW - 1)},
        "e2e": {"value": tokens_per_step * steps / float(e2e_s[0]), "unit": UNIT,
                "h2d_bytes_per_step": prompts_host.numel() * 4, "d2h_bytes_per_step": out_host.numel() * 4},
        "gpu_launches": (launches_prefill + launches_decode * (NEW - 1)) * steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "gemm_bf16_2cta_kernel (prefill QKV/O/gate-up/down shapes of this run)",
                     "achieved": achieved, "peak": peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": achieved / (peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]),
                     "peak_source": peaks["source"] + " (sustained cuBLAS bf16: the kernel runs inside a long step)",
                     # DRAM bytes of the four launches together: ncu measured 0.99 x the algorithmic 2(MK + NK + MN) bytes
                     # on a 4096 x 12288 x 4096 launch of this kernel (operands read once); scaled here by algorithmic bytes
                     "traffic": 0.99 * gemm_bytes, "traffic_unit": "bytes per set of four launches, scaled from an ncu capture"},
    }
    if not args.no_cpu_baseline and world == 1:
        v, desc, threads = cpu_generation_rate(cfg_kwargs, **CPU_SAMPLE)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}
    print(json.dumps(line), file=_JSON_OUT or sys.stdout, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
