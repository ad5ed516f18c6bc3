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
    """(result, ms per call): CUDA-event timed after warm-up (wall clock on CPU-only hosts), max
    over ranks when distributed."""
    import time
    gpu = torch.cuda.is_available()
    out = None
    for _ in range(warmups):
        out = func()
    if gpu:
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    if gpu:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    t0 = time.perf_counter()
    for _ in range(iters):
        out = func()
        if sync_per_iter and gpu:
            torch.cuda.synchronize()
    if gpu:
        stop.record()
        stop.synchronize()
        ms = start.elapsed_time(stop) / max(iters, 1)
    else:
        ms = (time.perf_counter() - t0) * 1e3 / max(iters, 1)
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], device="cuda" if gpu else "cpu")
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


# ------------------------------------------------------------------------------------------
# node-local group, fp8-friendly tensor constructors, int8 matmul, team split
# (reference: python/flux/testing/utils.py:98-124, 198-248, 280-290)
# ------------------------------------------------------------------------------------------
_TP_LOCAL_GROUP = None


def is_local_tp_group_initialized() -> bool:
    return _TP_LOCAL_GROUP is not None


def init_local_groups():
    """The group of the ranks on this node: the tensor-parallel group itself on one node (the
    only case this library runs), one new group per node otherwise."""
    global _TP_LOCAL_GROUP
    if _TP_LOCAL_GROUP is not None:
        raise RuntimeError("the node-local group exists already")
    tp = TP_GROUP()
    nnodes = NNODES()
    if nnodes == 1:
        _TP_LOCAL_GROUP = tp
        return _TP_LOCAL_GROUP
    lws = int(os.environ.get("LOCAL_WORLD_SIZE", 1))
    rank = dist.get_rank(tp)
    for n in range(nnodes):
        ranks = list(range(lws * n, lws * (n + 1)))
        pg = dist.new_group(ranks=ranks)
        if rank in ranks:
            _TP_LOCAL_GROUP = pg
    return _TP_LOCAL_GROUP


def _fp8(dtype) -> bool:
    return dtype in (torch.float8_e4m3fn, torch.float8_e5m2)


def _relaxed(fn, *args, **kwargs):
    # fill / copy kernels of 8-bit float types have no deterministic variant in torch
    from ..utils.util import with_torch_deterministic
    with with_torch_deterministic(False):
        return fn(*args, **kwargs)


def zeros_with_fp8(*args, **kwargs):
    return _relaxed(torch.zeros, *args, **kwargs)


def ones_with_fp8(*args, **kwargs):
    return _relaxed(torch.ones, *args, **kwargs)


def empty_non_determinisitc(*args, **kwargs):   # (spelling of the reference)
    return _relaxed(torch.empty, *args, **kwargs)


def rand_with_fp8(*args, dtype=None, **kwargs):
    if _fp8(dtype):
        return _relaxed(lambda: torch.rand(*args, dtype=torch.bfloat16, **kwargs).to(dtype))
    return torch.rand(*args, dtype=dtype, **kwargs)


def clone_with_fp8(tensor: torch.Tensor) -> torch.Tensor:
    return _relaxed(tensor.clone)


def all_gather_into_tensor_with_fp8(output_tensor, input_tensor, group=None, async_op=False):
    """NCCL has no 8-bit float type: such tensors travel as bytes."""
    if _fp8(input_tensor.dtype):
        return dist.all_gather_into_tensor(output_tensor.view(torch.uint8), input_tensor.view(torch.uint8),
                                           group=group, async_op=async_op)
    return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)


def matmul_int8(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] int8 @ b [K, N] int8 -> int32 (exact). ``torch._int_mm`` on CUDA needs more than 16
    rows, so short inputs are padded; on CPU the product is taken in int32 directly."""
    if not a.is_cuda:
        return a.to(torch.int32) @ b.to(torch.int32)
    M = a.shape[0]
    if M <= 16:
        return torch._int_mm(torch.nn.functional.pad(a, (0, 0, 0, 32 - M)), b)[:M]
    return torch._int_mm(a, b)


def nvshmem_split_team_2d(group_size: int):
    """(team of my ``group_size`` consecutive ranks, team of the ranks ``group_size`` apart)."""
    from ..parallel import teams
    return teams._nvshmem_team_split_2d(teams.TEAM_WORLD, group_size)


_GLOBAL_ARGS = {}


def set_global_args(**kwargs) -> None:
    """Key/value context that the perf log attaches to every record (reference:
    python/flux/testing/perf_db_helper.py)."""
    _GLOBAL_ARGS.update(kwargs)


def get_global_args() -> dict:
    return dict(_GLOBAL_ARGS)
