"""Runs the multi-rank worker (tests/dist_worker.py) on 2 / 4 / 8 GPUs of this node when it has
them: every fused op against NCCL-built PyTorch statements, one process per GPU."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, free_port

pytestmark = pytest.mark.gpu


def _run(world, what, extra_env=None):
    env = dict(os.environ, NCCL_DEBUG="WARN", FLUXB_WAIT_TIMEOUT_S="20")
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "dist_worker.py"), *what]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and "ALL OK" in r.stdout, r.stdout[-3000:] + "\n" + r.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ops_multi_gpu(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, ["dense", "blockscale", "ulysses", "moe", "coll"])


def test_rank_leaving_between_steps_is_detected():
    """Failure detection on the GPU without a fault: a rank stops launching, the others' bounded
    waits time out and report it. NVLS off in NCCL, plain peer stores in our kernels."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, ["failure"], {"NCCL_NVLS_ENABLE": "0"})
