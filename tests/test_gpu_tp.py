"""Tensor-parallel Qwen3 on 2 (and, where available, 4 / 8) GPUs of one node: greedy ids must equal the CPU oracle's
(and therefore the single-GPU run's) for every rank.  Skipped on boxes with one GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_oracle(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29500 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    # Also exercise the opt-in prefill that overlaps its all-reduces with the other half-batch's compute.  The decode
    # reduction has two forms (every rank gets every partial / row owners reduce and broadcast; the default switches
    # at 8 ranks): two ranks run both, four run the two-hop form too, eight their default.
    for hops in {2: ("1", "2"), 4: ("", "2")}.get(world, ("",)):
        env = dict(os.environ, TEENY_TP_OVERLAP="1")
        if hops:
            env["TEENY_TP_HOPS"] = hops
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
        assert f"TP{world} B4 S128 OK" in res.stdout and f"TP{world} B3 S40 OK" in res.stdout
        assert f"TP{world} sampling OK" in res.stdout
