"""Multi-GPU tests (need at least two GPUs; skipped otherwise): one process per GPU under torch.distributed.run."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(args, world=2, port=29541):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "multi_gpu_worker.py")] + args
    env = {"NCCL_NVLS_ENABLE": "0"}
    import os
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, **env})
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "multi-gpu worker ok" in done.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["nccl", "p2p", "p2p3"])
def test_kv_range_split_partials_cross_devices_and_merge(mode):
    _run(["kv_range", mode], port={"nccl": 29541, "p2p": 29542, "p2p3": 29544}[mode])


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_sequence_sharded_ranks_match_the_oracle():
    _run(["sequence"], port=29543)


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_kv_range_exchange_free_running_ranks_keep_their_steps_apart():
    _run(["kv_range_free_run"], port=29545)
