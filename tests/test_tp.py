"""Tensor parallelism: host-side plan and collective algebra on CPU (gloo, world size 2), the
real thing on 2+ GPUs."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, extra):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + os.getpid() % 500), os.path.join(HERE, "tp_worker.py")] + extra
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


def test_shard_plan_and_partial_sum_algebra_gloo_world2():
    r = _run(2, ["--cpu"])
    assert r.returncode == 0 and "tp cpu ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.gpu
def test_tensor_parallel_greedy_decode_matches_single_gpu():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(2, [])
    assert r.returncode == 0 and "tp gpu ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
