"""The example scripts run end to end on two CPU ranks (gloo, fp32 statements of the ops)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = [
    ("tp_mlp.py", ["--tokens", "64", "--hidden", "64", "--ffn", "128", "--iters", "2"], "TP2 MLP 64 tokens"),
    ("moe_layer.py", ["--tokens-per-rank", "16", "--hidden", "32", "--ffn", "24", "--experts", "4", "--topk", "2"],
     "MoE layer E=4 top2"),
    ("ulysses_attention.py", ["--seq", "32", "--heads", "4", "--head-dim", "8"], "Ulysses attention block seq 32"),
]


@pytest.mark.parametrize("script,args,expect", CASES)
def test_example_runs_on_cpu_ranks(script, args, expect):
    port = 29600 + (abs(hash(script)) % 200)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "examples", script), *args]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and expect in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
