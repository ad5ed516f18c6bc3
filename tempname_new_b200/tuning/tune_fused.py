"""Sweep the tile knobs of the fused ops on all ranks of a job and print the winners as tuning-file
entries - the role of the reference's ``tools/tune_gemm_rs.py``, ``tune_ag_gemm_kernel.py``,
``tune_gemm_a2a_transpose_kernel.py`` and ``tune_a2a_transpose_gemm_kernel.py``.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m tempname_new_b200.tuning.tune_fused --op gemm_rs --shape 8192,12288,49152

``--shape M,N,K`` is the whole problem: GEMM-RS computes [M, N] from K/W per rank, AG-GEMM computes
[M, N/W] from M/W rows per rank; for the Ulysses ops (``ulysses_pre`` / ``ulysses_post``) M is the
whole sequence (bs = 1), N x K the projection, ``--head-dim`` the head size. A candidate's time is
the maximum over ranks of a back-to-back loop (``--seconds`` long, so that the power cap and not the
boost clock of a short burst decides). The JSON lines that rank 0 prints can be collected into a
file named by ``FLUXB_TUNE_FILE``.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .table import candidates, override


def _timed(fn, seconds: float, dev) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    n = torch.tensor([max(5, int(seconds * 1e3 / max(s.elapsed_time(e), 1e-3)))], device=dev)
    dist.all_reduce(n, op=dist.ReduceOp.MAX)             # the same loop length on every rank
    iters = int(n.item())
    dist.barrier()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def tune(op_name: str, M: int, N: int, K: int, pg, dev, seconds: float = 0.5, head_dim: int = 128, cands=None):
    import tempname_new_b200 as flux
    W = dist.get_world_size(pg)
    seg_rows = 0
    if op_name == "gemm_rs":
        a = (torch.randn(M, K // W, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K // W, device=dev) * 0.02).bfloat16()
        op = flux.GemmRS(pg, 1, M, N, torch.bfloat16)
        key, seg_rows = (M, N, K // W), M // W
        run = lambda: op.forward(a, w)  # noqa: E731
    elif op_name == "ag_gemm":
        a = (torch.randn(M // W, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N // W, K, device=dev) * 0.02).bfloat16()
        op = flux.AGKernel(pg, 1, M, N // W, K, torch.bfloat16)
        out = torch.empty(M, N // W, device=dev, dtype=torch.bfloat16)
        key, seg_rows = (M, N // W, K), M // W
        run = lambda: op.forward(a, w, output=out)  # noqa: E731
    elif op_name == "ulysses_pre":
        x = (torch.randn(1, M // W, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        op = flux.GemmAllToAllTranspose(pg, 1, W, 1, M, K, head_dim, N, torch.bfloat16)
        key = (M // W, N, K)
        run = lambda: op.forward(x, w)  # noqa: E731
    elif op_name == "ulysses_post":
        nh = K // head_dim
        x = (torch.randn(1, nh // W, M, head_dim, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        op = flux.AllToAllTransposeGemm(pg, 1, W, 1, nh, M, head_dim, torch.bfloat16)
        key = (M // W, N, K)
        run = lambda: op.forward(x, w)  # noqa: E731
    else:
        raise ValueError("--op gemm_rs | ag_gemm | ulysses_pre | ulysses_post")
    res = []
    for knobs in (cands or candidates(*key, segmented_rows=seg_rows)):
        if op_name.startswith("ulysses") and knobs.get("tile_m", 0) == 512:
            continue                                    # the all-to-all modes run on 128 / 256-row tiles
        with override(key, knobs):
            ms = _timed(run, seconds, dev)
        op.check_status()
        res.append((ms, knobs))
    res.sort(key=lambda r: r[0])
    return {"op": op_name, "world": W, "key": list(key), "best": res[0][1], "ms": res[0][0],
            "all": [{"ms": r[0], **r[1]} for r in res]}


def main():
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm_rs", "ag_gemm", "ulysses_pre", "ulysses_post"])
    ap.add_argument("--shape", action="append", required=True, help="M,N,K of the whole problem")
    ap.add_argument("--seconds", type=float, default=0.5)
    ap.add_argument("--head-dim", type=int, default=128)
    args = ap.parse_args()
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    pg = dist.group.WORLD
    for s in args.shape:
        M, N, K = (int(v) for v in s.split(","))
        r = tune(args.op, M, N, K, pg, dev, args.seconds, args.head_dim)
        if dist.get_rank() == 0:
            print(json.dumps(r), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
