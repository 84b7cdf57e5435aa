"""Multi-GPU tests: each launches a torchrun job on all visible GPUs (2 to 8)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(script, nproc, timeout=420, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", str(nproc), os.path.join(HERE, script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_sharded_engine_multi_gpu():
    out = _launch("dist_sharded_check.py", min(torch.cuda.device_count(), 8))
    assert "sharded check ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_peer_collectives_multi_gpu():
    out = _launch("dist_tp_check.py", min(torch.cuda.device_count(), 8))
    assert "tp check ok" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_times_sharded_data_parallel_multi_gpu():
    """2-way tensor parallel x sharded data parallel.  With four or more GPUs visible: 4 ranks (2 x 2, the gradient
    reduction inside the data-parallel groups under the tensor-parallel controller); with two: one tensor-parallel
    group and single-rank data-parallel groups (the shard / replica noise ranges).  OPACUS_B200_2D_RANKS overrides
    (2, 4 or 8)."""
    n = torch.cuda.device_count()
    default = "4" if n >= 4 else "2"
    nproc = min(int(os.environ.get("OPACUS_B200_2D_RANKS", default)), n - n % 2)
    out = _launch("dist_tp_fsdp_check.py", nproc, TP_SIZE="2")
    assert "tp x fsdp check ok" in out
