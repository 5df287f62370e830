"""Tensor-parallel host logic on CPU: the Megatron sharding of teenygrad_b200.tp reproduces the unsharded layer
when the partial products are summed with a world-size-2 gloo all-reduce, and the vocabulary-parallel greedy pick
(local argmax + merge) equals a global argmax.  No GPU, no CUDA library calls."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from oracle import qwen3 as oq


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _reference_layer(cfg, sd, x):
    """o_proj(q|k|v slices mixed trivially) and the MLP of layer 0 on f32 copies: enough to exercise every shard."""
    p = "model.layers.0."
    f = {k: v.float() for k, v in sd.items() if k.startswith(p)}
    qkv = torch.cat([F.linear(x, f[p + "self_attn.q_proj.weight"]), F.linear(x, f[p + "self_attn.k_proj.weight"]),
                     F.linear(x, f[p + "self_attn.v_proj.weight"])], dim=-1)
    attn_like = torch.tanh(qkv[:, :cfg.num_q_heads * cfg.head_dim])
    o = F.linear(attn_like, f[p + "self_attn.o_proj.weight"])
    mlp = F.linear(F.silu(F.linear(x, f[p + "mlp.gate_proj.weight"])) * F.linear(x, f[p + "mlp.up_proj.weight"]),
                   f[p + "mlp.down_proj.weight"])
    return qkv, o, mlp


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from teenygrad_b200 import tp
    cfg = oq.OracleQwen3Config(1, 64, 4, 2, 128, 128, 512, tied=False)
    sd = oq.make_weights(cfg, 11)
    x = torch.randn(5, cfg.hidden, generator=torch.Generator().manual_seed(1))
    qkv_ref, o_ref, mlp_ref = _reference_layer(cfg, sd, x)
    sh = {k: v.float() for k, v in tp.shard_layer(sd, cfg, 0, rank, world).items()}
    D, hq, hkv, il = cfg.head_dim, cfg.num_q_heads // world, cfg.num_kv_heads // world, cfg.intermediate // world
    qkv = F.linear(x, sh["qkv"])
    q_ref = qkv_ref[:, rank * hq * D:(rank + 1) * hq * D]
    k_ref = qkv_ref[:, cfg.num_q_heads * D + rank * hkv * D: cfg.num_q_heads * D + (rank + 1) * hkv * D]
    ok = torch.allclose(qkv[:, :hq * D], q_ref, atol=1e-5) and torch.allclose(qkv[:, hq * D:(hq + hkv) * D], k_ref, atol=1e-5)
    o = F.linear(torch.tanh(qkv[:, :hq * D]), sh["o"])
    dist.all_reduce(o)
    gu = F.linear(x, sh["gate_up"])
    gu = gu.view(-1, il // 64, 2, 64)  # blocks of 64 gate channels followed by the same 64 up channels
    mlp = F.linear((F.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(-1, il), sh["down"])
    dist.all_reduce(mlp)
    ok = ok and torch.allclose(o, o_ref, atol=1e-4) and torch.allclose(mlp, mlp_ref, atol=1e-4)
    # vocabulary-parallel greedy pick
    head = tp.shard_head(sd, cfg, rank, world)
    hidden = torch.randn(3, cfg.hidden, generator=torch.Generator().manual_seed(2))
    logits = F.linear(hidden, head["lm_head"].float())
    logits[1, 0] = 50.0 if rank == 1 else logits[1, 0]          # winner on rank 1
    full = F.linear(hidden, sd["lm_head.weight"].float())
    full[1, cfg.vocab // world] = 50.0
    val, idx = logits.max(dim=-1)
    idx = idx + rank * (cfg.vocab // world)
    vals = [torch.empty_like(val) for _ in range(world)]
    idxs = [torch.empty_like(idx) for _ in range(world)]
    dist.all_gather(vals, val)
    dist.all_gather(idxs, idx)
    merged = tp.merge_argmax(torch.stack(vals), torch.stack(idxs))
    ok = ok and torch.equal(merged, full.argmax(dim=-1))
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_sharding_and_vocab_parallel_argmax_world2():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[0] and ret[1]


def test_merge_argmax_ties_pick_lowest_index():
    from teenygrad_b200 import tp
    vals = torch.tensor([[1.0, 5.0], [1.0, 4.0]])
    idx = torch.tensor([[7, 3], [2, 9]])
    assert tp.merge_argmax(vals, idx).tolist() == [2, 3]


def test_shard_shapes_8b_tp8():
    from teenygrad_b200 import tp
    cfg = oq.OracleQwen3Config(1, 4096, 32, 8, 128, 12288, 151936)
    sd = {f"model.layers.0.{n}": torch.empty(s, dtype=torch.bfloat16, device="meta") for n, s in {
        "self_attn.q_proj.weight": (4096, 4096), "self_attn.k_proj.weight": (1024, 4096),
        "self_attn.v_proj.weight": (1024, 4096), "self_attn.o_proj.weight": (4096, 4096),
        "mlp.gate_proj.weight": (12288, 4096), "mlp.up_proj.weight": (12288, 4096),
        "mlp.down_proj.weight": (4096, 12288), "input_layernorm.weight": (4096,),
        "post_attention_layernorm.weight": (4096,), "self_attn.q_norm.weight": (128,),
        "self_attn.k_norm.weight": (128,)}.items()}
    sh = tp.shard_layer(sd, cfg, 0, 3, 8)
    assert sh["qkv"].shape == (768, 4096) and sh["o"].shape == (4096, 512)
    assert sh["gate_up"].shape == (3072, 4096) and sh["down"].shape == (4096, 1536)


_FAKE_NCCL = r"""
/* Stand-in for libnccl.so.2 on a machine without GPUs: a communicator whose rendezvous never completes (the other
 * rank never arrives).  Records what the library under test does with it. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef int ncclResult_t;
enum { ncclSuccess = 0, ncclInProgress = 7 };
static int polls = 0;
static void note(const char* what) {
  const char* path = getenv("FAKE_NCCL_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (f) { fprintf(f, "%s polls=%d\n", what, polls); fclose(f); }
}
ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof(*id)); return ncclSuccess; }
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int n, ncclUniqueId id, int rank, void* config) {
  (void)n; (void)id; (void)rank;
  /* the blocking flag is the int behind size, magic and version in ncclConfig_t */
  note(((int*)((char*)config + sizeof(size_t)))[2] == 0 ? "init nonblocking" : "init blocking");
  *comm = (ncclComm_t)0x1234;
  return ncclInProgress;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* state) { (void)comm; ++polls; *state = ncclInProgress; return ncclSuccess; }
ncclResult_t ncclCommAbort(ncclComm_t comm) { note(comm == (ncclComm_t)0x1234 ? "abort guard" : "abort other"); return ncclSuccess; }
ncclResult_t ncclCommInitRank(ncclComm_t* c, int n, ncclUniqueId id, int r) { (void)c; (void)n; (void)id; (void)r; note("blocking init"); return 1; }
ncclResult_t ncclCommDestroy(ncclComm_t c) { (void)c; return ncclSuccess; }
ncclResult_t ncclAllReduce(void) { return 1; }
ncclResult_t ncclAllGather(void) { return 1; }
ncclResult_t ncclBroadcast(void) { note("broadcast"); return 1; }
ncclResult_t ncclGroupStart(void) { return ncclSuccess; }
ncclResult_t ncclGroupEnd(void) { return ncclSuccess; }
"""


def test_rendezvous_with_a_rank_that_never_arrives_times_out_and_aborts(tmp_path):
    """teeny_tp_init against a stand-in NCCL whose communicator never finishes its rendezvous (the peer rank exited
    before joining): the call must come back with TEENY_ERR_NCCL after the host timeout, having aborted the guard
    communicator, and must not have fallen into the blocking initialisation."""
    import shutil
    import subprocess
    import sys
    import time
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler for the NCCL stand-in")
    src, so, log = tmp_path / "fake_nccl.c", tmp_path / "libfake_nccl.so", tmp_path / "calls.log"
    src.write_text(_FAKE_NCCL)
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so), str(src)])
    code = (
        "import ctypes, sys, time\n"
        "from teenygrad_b200 import qwen3\n"
        "buf = (ctypes.c_ubyte * 128)()\n"
        "assert qwen3.lib.teeny_tp_unique_id(buf) == 0\n"
        "comm = ctypes.c_void_p()\n"
        "t0 = time.time()\n"
        "rc = qwen3.lib.teeny_tp_init(bytes(buf), 0, 2, ctypes.byref(comm))\n"
        "print('rc', rc, 'seconds', round(time.time() - t0, 2), 'comm', comm.value)\n"
    )
    env = dict(os.environ, TEENY_NCCL_LIB=str(so), TEENY_TP_INIT_TIMEOUT_MS="400", FAKE_NCCL_LOG=str(log),
               PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    t0 = time.time()
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "rc -6 " in res.stdout and "comm None" in res.stdout, res.stdout   # TEENY_ERR_NCCL, no context handed out
    seconds = float(res.stdout.split("seconds")[1].split()[0])
    assert 0.3 <= seconds < 5.0, res.stdout                                     # the timeout, not a hang and not at once
    calls = log.read_text().splitlines()
    assert calls[0].startswith("init nonblocking")
    assert calls[-1].startswith("abort guard") and "polls=0" not in calls[-1]   # polled, then aborted
    assert not any(c.startswith(("blocking init", "broadcast")) for c in calls)
