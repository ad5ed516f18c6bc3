"""Distributed set-up and data helpers for test scripts (reference:
``python/flux/testing/utils.py:49-283``)."""
from __future__ import annotations

import datetime
import os
import random
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

_TP_GROUP = None

# tolerances of the reference's op tests (test/python/gemm_rs/test_gemm_rs.py:588-594)
DTYPE_TOLERANCE = {
    torch.bfloat16: 2e-2, torch.float16: 1e-2, torch.float8_e4m3fn: 3e-2, torch.float8_e5m2: 3e-2,
    torch.int8: 2e-1, torch.float32: 1e-5,
}


def init_seed(seed: int = 0) -> None:
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":16:8")
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.manual_seed(3 + seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(3 + seed)
    torch.backends.cuda.matmul.allow_tf32 = False
    np.random.seed(3 + seed)
    random.seed(3 + seed)


def NNODES() -> int:
    return max(int(os.environ.get("WORLD_SIZE", 1)) // max(int(os.environ.get("LOCAL_WORLD_SIZE", 1)), 1), 1)


def initialize_distributed(backend: Optional[str] = None):
    """Create the default group (NCCL on GPUs, gloo otherwise), seed per rank and prepare
    symmetric memory; returns the tensor-parallel group (all ranks)."""
    global _TP_GROUP
    if _TP_GROUP is not None:
        return _TP_GROUP
    from ..parallel.symm import init_flux_shm
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, world_size=world, rank=rank,
                                timeout=datetime.timedelta(seconds=1800), **kw)
    _TP_GROUP = dist.new_group(ranks=list(range(world)), backend=backend)
    init_seed(rank)
    init_flux_shm(_TP_GROUP)
    return _TP_GROUP


def TP_GROUP():
    if _TP_GROUP is None:
        raise RuntimeError("call initialize_distributed() first")
    return _TP_GROUP


def _make(shape: Sequence[int], dtype: torch.dtype, scale_offset: Tuple[float, float], device) -> torch.Tensor:
    scale, offset = scale_offset
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return ((torch.rand(shape, device=device) * 2 - 1) * scale + offset).to(dtype)
    if dtype in (torch.int8, torch.int32):
        return torch.randint(-127, 128, shape, device=device).to(dtype)
    return ((torch.rand(shape, dtype=torch.float32, device=device) * 2 - 1) * scale + offset).to(dtype)


def generate_data(configs: List[Tuple[Sequence[int], torch.dtype, Tuple[float, float]]], device=None):
    """Yield lists of tensors forever, one per ``(shape, dtype, (scale, offset))`` entry: uniform
    in [offset - scale, offset + scale] (the reference scales by 0.01 * (rank + 1))."""
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    while True:
        yield [None if c is None else _make(*c, device=device) for c in configs]


def run_perf(expname: str, warmups: int, iters: int, func: Callable, sync_per_iter: bool = False):
    """(result, ms per call): CUDA-event timed after warm-up, max over ranks when distributed."""
    out = None
    for _ in range(warmups):
        out = func()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        out = func()
        if sync_per_iter:
            torch.cuda.synchronize()
    stop.record()
    stop.synchronize()
    ms = start.elapsed_time(stop) / max(iters, 1)
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return out, ms


def bitwise_eq(x: torch.Tensor, y: torch.Tensor) -> bool:
    from ..ops.misc import bitwise_check
    return bitwise_check(x, y)


def split_torch_process_group(pg, group_size: int):
    """Cut ``pg`` into consecutive sub-groups of ``group_size`` ranks; returns this rank's."""
    world, rank = dist.get_world_size(pg), dist.get_rank(pg)
    if world % group_size:
        raise ValueError("group_size must divide the group")
    ranks = dist.get_process_group_ranks(pg)
    mine = None
    for start in range(0, world, group_size):
        sub = dist.new_group(ranks=ranks[start:start + group_size])
        if start <= rank < start + group_size:
            mine = sub
    return mine
