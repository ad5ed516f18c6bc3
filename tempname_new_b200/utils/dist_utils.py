"""Process-group bootstrap helpers (reference: ``python/flux/dist_utils.py:25-90``)."""
from __future__ import annotations

import datetime
import os
import random
from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist


class DistEnv:
    def __init__(self, deterministic: bool = True, backend: Optional[str] = None):
        self.RANK = int(os.environ.get("RANK", 0))
        self.LOCAL_RANK = int(os.environ.get("LOCAL_RANK", 0))
        self.LOCAL_WORLD_SIZE = int(os.environ.get("LOCAL_WORLD_SIZE", 1))
        self.WORLD_SIZE = int(os.environ.get("WORLD_SIZE", 1))
        self.NNODES = max(self.WORLD_SIZE // max(self.LOCAL_WORLD_SIZE, 1), 1)
        self.backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if not dist.is_initialized():
            kw = {}
            if self.backend == "nccl":
                torch.cuda.set_device(self.LOCAL_RANK)
                kw["device_id"] = torch.device("cuda", self.LOCAL_RANK)
            dist.init_process_group(self.backend, world_size=self.WORLD_SIZE, rank=self.RANK,
                                    timeout=datetime.timedelta(seconds=1800), **kw)
        if deterministic:
            self.setup_deterministic(self.RANK)

    def setup_deterministic(self, seed: int) -> None:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":16:8")
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)
        torch.backends.cuda.matmul.allow_tf32 = False
        np.random.seed(seed)
        random.seed(seed)

    def get_world(self):
        return dist.group.WORLD

    def new_group(self, ranks):
        return dist.new_group(ranks=ranks, backend=self.backend)


_ENV: Optional[DistEnv] = None


def get_dist_env(deterministic: bool = True) -> DistEnv:
    global _ENV
    if _ENV is None:
        _ENV = DistEnv(deterministic)
    return _ENV


def exec_in_rank_order(group, func: Callable) -> None:
    """Run ``func`` on one rank after the other (ordered debug printing)."""
    for r in range(dist.get_world_size(group)):
        if r == dist.get_rank(group):
            func()
        dist.barrier(group=group)
        if torch.cuda.is_available():
            torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------
# Node-level process groups of a tensor-parallel group that spans several nodes (reference:
# python/flux/gemm_rs_sm80.py:31-84 and python/flux/ag_kernel_internode.py:32-73, where the
# multi-node GEMM-RS / AG-GEMM variants use them). The fused ops of this library run inside one
# node; the groups are plain torch groups and are provided so that scripts which build them keep
# working (a job can still shard its outer dimension across nodes with them).
# ------------------------------------------------------------------------------------------
_NODE_GROUPS = {}


def _node_group(kind: str, tp_group, nnodes: int):
    key = (kind, id(tp_group), nnodes)
    if key in _NODE_GROUPS:
        return _NODE_GROUPS[key]
    tp_world = dist.get_world_size(tp_group)
    world = dist.get_world_size()
    if tp_world % nnodes or world % tp_world:
        raise ValueError(f"{tp_world} ranks do not divide over {nnodes} nodes (world {world})")
    local = tp_world // nnodes
    me = dist.get_rank()
    mine = None
    if kind == "intra":
        sets = [list(range(tp0 + n * local, tp0 + (n + 1) * local))
                for tp0 in range(0, world, tp_world) for n in range(nnodes)]
    else:
        sets = [[tp0 + n * local + lr for n in range(nnodes)]
                for tp0 in range(0, world, tp_world) for lr in range(local)]
    for ranks in sets:                       # every rank creates every group: new_group is collective
        g = dist.new_group(ranks=ranks)
        if me in ranks:
            mine = g
    _NODE_GROUPS[key] = mine
    return mine


def get_intra_node_pg_group(tp_group, nnodes: int):
    """The ranks of ``tp_group`` that share this rank's node."""
    return _node_group("intra", tp_group, nnodes)


def get_intra_node_ag_group(tp_group, nnodes: int):
    return _node_group("intra", tp_group, nnodes)


def get_inter_node_ag_group(tp_group, nnodes: int):
    """The ranks of ``tp_group`` with this rank's local index, one per node."""
    return _node_group("inter", tp_group, nnodes)


_INTER_NODE_RS_GROUP = None


def initialize_inter_node_rs_group(tp_group, nnodes: int) -> None:
    global _INTER_NODE_RS_GROUP
    if _INTER_NODE_RS_GROUP is None:
        _INTER_NODE_RS_GROUP = _node_group("inter", tp_group, nnodes)


def get_inter_node_rs_group():
    if _INTER_NODE_RS_GROUP is None:
        raise RuntimeError("call initialize_inter_node_rs_group(tp_group, nnodes) first")
    return _INTER_NODE_RS_GROUP
