"""Tensor-parallel MLP block (AG+GEMM -> GEMM+RS) with sequence-sharded activations.

    ./launch.sh examples/tp_mlp.py --tokens 8192 --hidden 12288 --ffn 49152
"""
import argparse

import torch

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
mlp = TPMLP(args.hidden, args.ffn, pg, dtype=torch.bfloat16, device="cuda").requires_grad_(False)
x = torch.randn(args.tokens // world, args.hidden, device="cuda").bfloat16()
with torch.no_grad():
    y, ms = run_perf("tp_mlp", 3, args.iters, lambda: mlp(x))
flops = 4.0 * args.tokens * args.hidden * args.ffn
if rank == 0:
    print(f"TP{world} MLP {args.tokens} tokens: {ms:.3f} ms/step, {flops / ms / 1e9:.0f} TFLOP/s over the job, "
          f"output {tuple(y.shape)}")
