"""Per-call option records of the reference API (``src/pybind/ths_op.cc:148-203``).

On an NVSwitch node there is one transport (direct peer access at full bandwidth to every
peer), so the ring / copy-engine / NUMA knobs select nothing here: they are accepted and kept
so that code written against the reference runs unchanged."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional


class AGRingMode(enum.IntEnum):
    All2All = 0
    Ring1D = 1
    Ring2D = 2


class RingMode(enum.IntEnum):
    All2All = 0
    Ring1D = 1
    Ring2D = 2


class A2ARingMode(enum.IntEnum):
    All2All = 0
    Ring1D = 1
    Ring2D = 2


class PreAttnAllToAllCommOp(enum.IntEnum):
    A2ATranspose = 0
    QKVPackA2A = 1


def get_default_ag_ring_mode() -> AGRingMode:
    return AGRingMode.All2All


def get_default_rs_ring_mode() -> RingMode:
    return RingMode.All2All


def get_default_a2a_ring_mode() -> A2ARingMode:
    return A2ARingMode.All2All


@dataclass
class AllGatherOption:
    input_buffer_copied: Optional[bool] = None
    use_read: Optional[bool] = None
    mode: Optional[AGRingMode] = None
    fuse_sync: Optional[bool] = None
    use_cuda_core_local: Optional[bool] = None
    use_cuda_core_ag: Optional[bool] = None


@dataclass
class ReduceScatterOption:
    use_barrier_queue: Optional[bool] = None
    use_1d_ring: Optional[bool] = None
    use_p2p_read: Optional[bool] = None
    use_cudaMemcpyAsync: Optional[bool] = None
    use_gemmk: Optional[bool] = None
    per_tile_flags: Optional[bool] = None
    n_split: Optional[int] = None
    num_blocks: Optional[int] = None
    ring_mode: Optional[RingMode] = None


@dataclass
class AllToAllOption:
    input_buffer_copied: Optional[bool] = None
    use_cuda_core: Optional[bool] = None
    fuse_sync: Optional[bool] = None
    use_read: Optional[bool] = None
    skip_barrier: Optional[bool] = None
    mode: Optional[A2ARingMode] = None
