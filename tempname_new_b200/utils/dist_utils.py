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
