"""Sweep the tile knobs of the fused ops (GEMM + reduce-scatter, all-gather + GEMM) on all ranks of
a job and print the winners as tuning-file entries - the role of the reference's
``tools/tune_gemm_rs.py`` and ``tools/tune_ag_gemm_kernel.py``.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m tempname_new_b200.tuning.tune_fused --op gemm_rs --shape 8192,12288,49152

``--shape M,N,K`` is the whole problem: GEMM-RS computes [M, N] from K/W per rank, AG-GEMM
computes [M, N/W] from M/W rows per rank. A candidate's time is the maximum over ranks. The JSON
lines that rank 0 prints can be collected into a file named by ``FLUXB_TUNE_FILE``.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .table import override

CANDIDATES = [(2, 256, 8), (2, 256, 4), (2, 256, 2), (1, 128, 16), (1, 128, 8)]


def _timed(fn, iters: int, warmup: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def tune(op_name: str, M: int, N: int, K: int, pg, dev, iters: int = 10, candidates=None):
    import tempname_new_b200 as flux
    W = dist.get_world_size(pg)
    if op_name == "gemm_rs":
        a = (torch.randn(M, K // W, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K // W, device=dev) * 0.02).bfloat16()
        op = flux.GemmRS(pg, 1, M, N, torch.bfloat16)
        key = (M, N, K // W)
        run = lambda: op.forward(a, w)  # noqa: E731
    elif op_name == "ag_gemm":
        a = (torch.randn(M // W, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N // W, K, device=dev) * 0.02).bfloat16()
        op = flux.AGKernel(pg, 1, M, N // W, K, torch.bfloat16)
        out = torch.empty(M, N // W, device=dev, dtype=torch.bfloat16)
        key = (M, N // W, K)
        run = lambda: op.forward(a, w, output=out)  # noqa: E731
    else:
        raise ValueError("--op gemm_rs | ag_gemm")
    res = []
    for cg, bn, gm in (candidates or CANDIDATES):
        knobs = {"cta_group": cg, "tile_n": bn, "group_m": gm}
        with override(key, knobs):
            ms = _timed(run, iters, 3, dev)
        op.check_status()
        res.append((ms, knobs))
    res.sort(key=lambda r: r[0])
    return {"op": op_name, "key": list(key), "best": res[0][1], "ms": res[0][0],
            "all": [{"ms": r[0], **r[1]} for r in res]}


def main():
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm_rs", "ag_gemm"])
    ap.add_argument("--shape", action="append", required=True, help="M,N,K of the whole problem")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    pg = dist.group.WORLD
    for s in args.shape:
        M, N, K = (int(v) for v in s.split(","))
        r = tune(args.op, M, N, K, pg, dev, args.iters)
        if dist.get_rank() == 0:
            print(json.dumps(r), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
