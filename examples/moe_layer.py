"""One MoE layer (router -> layer 0 -> SwiGLU -> layer 1) on the fused ops, expert parallel over
all GPUs (reference: examples/moe_flux_only.py).

    ./launch.sh examples/moe_layer.py --tokens-per-rank 8192 --experts 64 --topk 8
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout

import tempname_new_b200 as flux
from tempname_new_b200.testing import gate_func, initialize_distributed, run_perf

ap = argparse.ArgumentParser()
ap.add_argument("--tokens-per-rank", type=int, default=2048)
ap.add_argument("--hidden", type=int, default=4096)
ap.add_argument("--ffn", type=int, default=1536)
ap.add_argument("--experts", type=int, default=64)
ap.add_argument("--topk", type=int, default=8)
args = ap.parse_args()

pg = initialize_distributed()
rank, world = pg.rank(), pg.size()
# GPUs run the sm_100a kernels in bf16; without one the same script runs the CPU statements in fp32
DEV, DT = ("cuda", torch.bfloat16) if torch.cuda.is_available() else ("cpu", torch.float32)
tokens = args.tokens_per_rank * world
E, topk, H, F = args.experts, args.topk, args.hidden, args.ffn
E_loc = E // world
env = flux.DistEnvTPWithEP(pg, 1, None, ep_size=world)
layer0 = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(tokens, H, 2 * F, E, topk, DT))
layer1 = flux.GemmGroupedV3GatherRS(E, tokens * topk, H, topk, rank, world, 1, world, tp_group=pg, dtype=DT)
torch.manual_seed(0)                                           # router weights identical on all ranks
router = (torch.randn(E, H, device=DEV) * 0.02).to(DT)
torch.manual_seed(1 + rank)
w_gate_up = (torch.randn(E_loc, 2 * F, H, device=DEV) * 0.02).to(DT)
w_down = (torch.randn(E_loc, H, F, device=DEV) * 0.02).to(DT)
x = torch.randn(args.tokens_per_rank, H, device=DEV).to(DT)


def layer():
    # routing needs every rank's choices: gather the (small) router outputs
    chosen, gate = gate_func(x, router, topk)
    all_chosen = torch.empty(tokens, topk, dtype=torch.int32, device=DEV)
    all_gate = torch.empty(tokens, topk, dtype=torch.float32, device=DEV)
    torch.distributed.all_gather_into_tensor(all_chosen, chosen.contiguous(), group=pg)
    torch.distributed.all_gather_into_tensor(all_gate, gate.float().contiguous(), group=pg)
    splits, offsets, scatter, gather, tki = flux.moe_index_build(all_chosen, E)
    lo, hi = offsets[rank * E_loc], offsets[(rank + 1) * E_loc]
    rows = int(hi - lo)                                        # the only host sync: sizing the buffers
    h = torch.empty(rows, 2 * F, dtype=DT, device=DEV)
    layer0.forward(x, w_gate_up, splits, scatter, outputs_buf=h)
    act = torch.nn.functional.silu(h[:, :F].float()).mul_(h[:, F:].float()).to(DT)
    row_gate = all_gate.reshape(-1)[gather.long() * topk + tki.long()][int(lo):int(hi)].contiguous()
    return layer1.forward_gather_rs(act, w_down, splits, scatter.reshape(-1), output_vec_scale=row_gate)


y, ms = run_perf("moe_layer", 2, 5, layer)
if rank == 0:
    print(f"MoE layer E={E} top{topk} hidden {H} ffn {F}, {args.tokens_per_rank} tokens/rank on {world} GPUs: "
          f"{ms:.3f} ms, output {tuple(y.shape)}")
