"""Ulysses sequence-parallel attention block: fused QKV projection + seq->heads all-to-all, SDPA on
the local heads, fused heads->seq all-to-all + output projection.

    ./launch.sh examples/ulysses_attention.py --seq 32768 --heads 32 --head-dim 128
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout

import tempname_new_b200 as flux
from tempname_new_b200.testing import initialize_distributed, run_perf

ap = argparse.ArgumentParser()
ap.add_argument("--seq", type=int, default=8192)
ap.add_argument("--heads", type=int, default=32)
ap.add_argument("--head-dim", type=int, default=128)
ap.add_argument("--bs", type=int, default=1)
args = ap.parse_args()

pg = initialize_distributed()
rank, world = pg.rank(), pg.size()
# GPUs run the sm_100a kernels in bf16; without one the same script runs the CPU statements in fp32
DEV, DT = ("cuda", torch.bfloat16) if torch.cuda.is_available() else ("cpu", torch.float32)
hidden = args.heads * args.head_dim
nh3 = 3 * args.heads                                           # q, k, v heads (gqa = 1: equal counts)
pre = flux.GemmAllToAllTranspose(pg, 1, world, args.bs, args.seq, hidden, args.head_dim, nh3 * args.head_dim,
                                 DT, gqa=1, comm_op=flux.PreAttnAllToAllCommOp.QKVPackA2A)
post = flux.AllToAllTransposeGemm(pg, 1, world, args.bs, args.heads, args.seq, args.head_dim, DT,
                                  a2a_only=True)
w_qkv = (torch.randn(nh3 * args.head_dim, hidden, device=DEV) * 0.02).to(DT)
w_o = (torch.randn(hidden, hidden, device=DEV) * 0.02).to(DT)
x = torch.randn(args.bs, args.seq // world, hidden, device=DEV).to(DT)


def block():
    q, k, v = pre.forward(x, w_qkv)                            # each [bs, seq, heads/W, hd]
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    return post.forward(o.transpose(1, 2).contiguous(), w_o)   # [bs, seq/W, hidden]


y, ms = run_perf("ulysses", 2, 5, block)
if rank == 0:
    print(f"Ulysses attention block seq {args.seq}, {args.heads} x {args.head_dim} on {world} GPUs: {ms:.3f} ms, "
          f"output {tuple(y.shape)}")
