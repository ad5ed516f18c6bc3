"""Process-group descriptors passed to the MoE ops (reference: ``DistEnvTP``,
``DistEnvTPWithEP``, ``MoeArguments`` in ``src/ths_op/ths_op.cc`` and
``include/flux/ths_op/ths_op.h``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


class DistEnvTP:
    """Tensor-parallel group of one node (``nnodes`` is kept for API compatibility; this
    library targets a single NVSwitch domain, so it must be 1)."""

    def __init__(self, tp_group=None, nnodes: int = 1):
        if nnodes != 1:
            raise NotImplementedError("multi-node groups are outside the NVSwitch domain this library targets")
        self.tp_group = tp_group if tp_group is not None else dist.group.WORLD
        self.nnodes = nnodes
        self.rank = dist.get_rank(self.tp_group)
        self.world_size = dist.get_world_size(self.tp_group)
        self.local_rank = self.rank
        self.local_world_size = self.world_size

    def __repr__(self) -> str:
        return f"DistEnvTP(rank={self.rank}, world_size={self.world_size}, nnodes={self.nnodes})"


class DistEnvTPWithEP(DistEnvTP):
    """TP group that is further cut into expert-parallel groups: ``ep_size`` consecutive
    blocks of ``ffn_tp_size = world / ep_size`` ranks; rank r has ``ep_rank = r // ffn_tp_size``
    and ``ffn_tp_rank = r % ffn_tp_size`` (reference: ``src/ths_op/ths_op.cc:334-347``)."""

    def __init__(self, tp_group=None, nnodes: int = 1, ep_group=None, ep_size: Optional[int] = None):
        super().__init__(tp_group, nnodes)
        if ep_size is None:
            ep_size = dist.get_world_size(ep_group) if ep_group is not None else 1
        if self.world_size % ep_size != 0:
            raise ValueError("ep_size must divide the TP world size")
        self.ep_group = ep_group
        self.ep_size = ep_size
        self.ffn_tp_size = self.world_size // ep_size
        self.ep_rank = self.rank // self.ffn_tp_size
        self.ffn_tp_rank = self.rank % self.ffn_tp_size

    def __repr__(self) -> str:
        return (f"DistEnvTPWithEP(rank={self.rank}, world_size={self.world_size}, ep_size={self.ep_size}, "
                f"ep_rank={self.ep_rank}, ffn_tp_size={self.ffn_tp_size}, ffn_tp_rank={self.ffn_tp_rank})")


@dataclass
class MoeArguments:
    max_ntokens: int
    hidden: int
    ffn_hidden: int
    nexperts: int
    topk: int
    input_dtype: torch.dtype
    output_dtype: Optional[torch.dtype] = None

    def __post_init__(self):
        if self.output_dtype is None:
            # 8-bit inputs produce 16-bit results (the kernels' epilogues write bf16 / fp16 only)
            self.output_dtype = self.input_dtype if self.input_dtype.itemsize > 1 else torch.bfloat16
