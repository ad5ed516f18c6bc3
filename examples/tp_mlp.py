"""Tensor-parallel MLP block (AG+GEMM -> GEMM+RS) with sequence-sharded activations.

    ./launch.sh examples/tp_mlp.py --tokens 8192 --hidden 12288 --ffn 49152
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout

import tempname_new_b200 as flux
from tempname_new_b200.models.tp_mlp import TPMLP
from tempname_new_b200.testing import initialize_distributed, run_perf

ap = argparse.ArgumentParser()
ap.add_argument("--tokens", type=int, default=8192)
ap.add_argument("--hidden", type=int, default=4096)
ap.add_argument("--ffn", type=int, default=16384)
ap.add_argument("--iters", type=int, default=20)
args = ap.parse_args()

pg = initialize_distributed()
rank, world = pg.rank(), pg.size()
# GPUs run the sm_100a kernels in bf16; without one the same script runs the CPU statements in fp32
DEV, DT = ("cuda", torch.bfloat16) if torch.cuda.is_available() else ("cpu", torch.float32)
mlp = TPMLP(args.hidden, args.ffn, pg, dtype=DT, device=DEV).requires_grad_(False)
x = torch.randn(args.tokens // world, args.hidden, device=DEV).to(DT)
with torch.no_grad():
    y, ms = run_perf("tp_mlp", 3, args.iters, lambda: mlp(x))
flops = 4.0 * args.tokens * args.hidden * args.ffn
if rank == 0:
    print(f"TP{world} MLP {args.tokens} tokens: {ms:.3f} ms/step, {flops / ms / 1e9:.0f} TFLOP/s over the job, "
          f"output {tuple(y.shape)}")
