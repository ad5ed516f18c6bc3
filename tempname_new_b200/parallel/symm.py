"""Symmetric memory over one node: every rank allocates the same-sized block and can address
every peer's block directly.

* CUDA ranks: ``cudaMalloc`` + CUDA IPC handles exchanged over the process group, opened
  with lazy peer access; kernels then use plain peer loads/stores over NVLink/NVSwitch.
* CPU ranks (``gloo``, used by the plumbing and failure-detection tests): one file per rank
  under ``/dev/shm`` mapped shared by every rank, so the same ownership rules and flag
  protocols can be exercised without a GPU.

Reference: ``src/ths_op/flux_shm.cc`` (``cudaipc_create_tensor_list``, ``init_flux_shm``,
``GroupBarrier``) and ``src/cuda/cudaipc_barrier_all.cu``. NVSHMEM, ring mode and the pinned
``/dev/shm`` staging of the reference have no counterpart: NVSwitch gives every pair of GPUs a
direct path.
"""
from __future__ import annotations

import ctypes
import math
import os
import time
import uuid
import weakref
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native

_ELEM = {
    torch.uint8: 1, torch.int8: 1, torch.float8_e4m3fn: 1, torch.float8_e5m2: 1,
    torch.bfloat16: 2, torch.float16: 2, torch.int16: 2,
    torch.float32: 4, torch.int32: 4, torch.int64: 8, torch.float64: 8,
}


class FluxTimeoutError(RuntimeError):
    """A bounded wait (device flag, CPU flag or barrier) ran out of time."""


class _SymmHandle:
    """Owns one rank's symmetric block and its peer mappings; frees them when the last holder
    (the ``SymmBuffer`` or any tensor viewing its memory) is gone. Views keep this object alive,
    not the ``SymmBuffer`` itself, so a dropped buffer is collected by reference counting."""

    def __init__(self, is_cuda: bool, own_ptr: int, opened: Sequence[int]):
        self._fin = weakref.finalize(self, SymmBuffer._finalize, is_cuda, own_ptr, list(opened))

    @property
    def alive(self) -> bool:
        return self._fin.alive


class _CudaRaw:
    """``__cuda_array_interface__`` carrier for a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
        }
        self._owner = owner


def _group_ranks(pg) -> List[int]:
    return dist.get_process_group_ranks(pg)


def _is_cuda_group(pg) -> bool:
    return torch.cuda.is_available() and "nccl" in str(dist.get_backend(pg)).lower()


class SymmBuffer:
    """One symmetric allocation of ``nbytes`` bytes per rank.

    ``ptrs[r]`` is the address of rank r's block in this process; ``local`` is this rank's
    block as a flat ``uint8`` tensor; ``view(r, dtype, shape)`` gives a typed tensor over rank
    r's block (CUDA peers are materialised on demand).
    """

    def __init__(self, nbytes: int, pg=None, device: Optional[torch.device] = None):
        pg = pg if pg is not None else dist.group.WORLD
        self.pg = pg
        self.rank = dist.get_rank(pg)
        self.world = dist.get_world_size(pg)
        self.nbytes = int(math.ceil(max(nbytes, 16) / 256) * 256)
        self.is_cuda = _is_cuda_group(pg) if device is None else device.type == "cuda"
        self.ptrs: List[int] = [0] * self.world
        self._views: Dict[int, torch.Tensor] = {}
        self._opened: List[int] = []
        self._own_ptr = 0
        self._closed = False
        self._handle: Optional[_SymmHandle] = None
        if self.is_cuda:
            self.device = device or torch.device("cuda", torch.cuda.current_device())
            self._alloc_cuda()
        else:
            self.device = torch.device("cpu")
            self._alloc_shm()
            self._handle = _SymmHandle(False, 0, [])

    # ------------------------------------------------------------------ CUDA IPC
    def _alloc_cuda(self) -> None:
        lib = _native.lib()
        with torch.cuda.device(self.device):
            ptr = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            _native.check(lib.fluxb_symm_alloc(ctypes.c_uint64(self.nbytes), ctypes.byref(ptr), handle),
                          "symmetric allocation")
            self._own_ptr = int(ptr.value)
            mine = (os.getpid(), bytes(handle), self.nbytes)
            gathered: List = [None] * self.world
            dist.all_gather_object(gathered, mine, group=self.pg)
            for r, (pid, h, nb) in enumerate(gathered):
                if nb != self.nbytes:
                    raise ValueError(f"rank {r} allocated {nb} bytes, this rank {self.nbytes}: "
                                     "symmetric allocations must match on every rank")
                if r == self.rank:
                    self.ptrs[r] = self._own_ptr
                    continue
                p = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                _native.check(lib.fluxb_symm_open(buf, ctypes.byref(p)), f"opening rank {r}'s block")
                self.ptrs[r] = int(p.value)
                self._opened.append(int(p.value))
        self._handle = _SymmHandle(True, self._own_ptr, self._opened)
        self._views[self.rank] = torch.as_tensor(
            _CudaRaw(self._own_ptr, self.nbytes, self._handle), device=self.device)

    # ------------------------------------------------------------------ /dev/shm
    def _alloc_shm(self) -> None:
        tag = [uuid.uuid4().hex if self.rank == 0 else None]
        dist.broadcast_object_list(tag, src=_group_ranks(self.pg)[0], group=self.pg)
        base = f"/dev/shm/fluxb_{tag[0]}"
        self._paths = [f"{base}_{r}" for r in range(self.world)]
        mine = torch.from_file(self._paths[self.rank], shared=True, size=self.nbytes, dtype=torch.uint8)
        mine.zero_()
        dist.barrier(group=self.pg)
        for r in range(self.world):
            t = mine if r == self.rank else torch.from_file(
                self._paths[r], shared=True, size=self.nbytes, dtype=torch.uint8)
            self._views[r] = t
            self.ptrs[r] = t.data_ptr()
        dist.barrier(group=self.pg)
        try:  # every rank holds its mappings now; the names can go
            os.unlink(self._paths[self.rank])
        except OSError:
            pass

    @staticmethod
    def _finalize(is_cuda: bool, own_ptr: int, opened: Sequence[int]) -> None:
        if not is_cuda or own_ptr == 0:
            return
        try:
            lib = _native.lib()
            for p in opened:
                lib.fluxb_symm_close(ctypes.c_void_p(p))
            lib.fluxb_symm_free(ctypes.c_void_p(own_ptr))
        except Exception:
            pass

    # ------------------------------------------------------------------ views
    @property
    def local(self) -> torch.Tensor:
        return self._views[self.rank]

    def flat(self, r: int) -> torch.Tensor:
        if r not in self._views:
            self._views[r] = torch.as_tensor(_CudaRaw(self.ptrs[r], self.nbytes, self._handle), device=self.device)
        return self._views[r]

    def view(self, r: int, dtype: torch.dtype, shape: Sequence[int], offset_bytes: int = 0) -> torch.Tensor:
        n = int(math.prod(shape)) * _ELEM[dtype]
        if offset_bytes + n > self.nbytes:
            raise ValueError("view exceeds the symmetric block")
        return self.flat(r)[offset_bytes:offset_bytes + n].view(dtype).view(*shape)

    def ptr(self, r: int, offset_bytes: int = 0) -> int:
        return self.ptrs[r] + offset_bytes


_INITIALISED: "weakref.WeakSet" = weakref.WeakSet()


def init_flux_shm(pg=None) -> None:
    """Prepare symmetric memory for ``pg`` (reference: ``flux.init_flux_shm``).

    CUDA IPC and ``/dev/shm`` need no global bootstrap, so this only checks that every pair of
    GPUs in the group has peer access and fails early otherwise.
    """
    pg = pg if pg is not None else dist.group.WORLD
    if _is_cuda_group(pg):
        lib = _native.lib()
        dev = torch.cuda.current_device()
        devs: List = [None] * dist.get_world_size(pg)
        dist.all_gather_object(devs, dev, group=pg)
        for peer in devs:
            if peer == dev:
                continue
            ok = ctypes.c_int(0)
            _native.check(lib.fluxb_can_access_peer(dev, peer, ctypes.byref(ok)), "peer access query")
            if not ok.value:
                raise RuntimeError(f"GPU {dev} cannot access GPU {peer}: symmetric memory needs P2P")


def create_tensor_list(shape: Sequence[int], dtype: torch.dtype, pg=None, ring_mode: bool = False,
                       init_zero: bool = False) -> List[torch.Tensor]:
    """Symmetric tensors, one per rank of ``pg``; entry ``rank`` is local memory, the others
    are views of the peers' memory (reference: ``flux.create_tensor_list``). Blocks start
    zeroed, so ``init_zero`` is accepted for compatibility; ``ring_mode`` is ignored."""
    nbytes = int(math.prod(shape)) * _ELEM[dtype]
    buf = SymmBuffer(nbytes, pg)
    out = [buf.view(r, dtype, shape) for r in range(buf.world)]
    for t in out:
        t._fluxb_symm = buf  # keep the allocation alive as long as any view lives
    return out


def create_tensor(shape: Sequence[int], dtype: torch.dtype, pg=None) -> torch.Tensor:
    """This rank's tensor of a symmetric allocation (reference: ``flux.create_tensor``,
    python/flux/cpp_mod.pyi:31); the peers' views stay reachable through ``t._fluxb_symm``."""
    ts = create_tensor_list(shape, dtype, pg)
    return ts[ts[0]._fluxb_symm.rank]


# the reference exports the same allocator under a second name (cpp_mod.pyi:35-37)
flux_create_shm_tensor_list = create_tensor_list


class GroupBarrier:
    """Barrier over the ranks of ``pg`` that runs on the GPU stream (CPU groups: in shared
    memory). Flags carry the call number, so no reset pass is needed between calls and every
    wait is bounded (reference: ``flux.GroupBarrier``, which resets flags with CAS and spins
    without limit)."""

    def __init__(self, process_group=None, ring_mode: bool = False, timeout_s: float = 10.0):
        self.pg = process_group if process_group is not None else dist.group.WORLD
        self.buf = SymmBuffer(256, self.pg)
        self.rank, self.world = self.buf.rank, self.buf.world
        self.epoch = 0
        self.timeout_s = timeout_s
        if self.buf.is_cuda:
            self.status = torch.zeros(4, dtype=torch.int32, device=self.buf.device)
            self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.buf.ptrs)
        else:
            self._flags = [self.buf.view(r, torch.int32, (self.world,)) for r in range(self.world)]

    def barrier_all(self, stream: Optional[int] = None) -> None:
        self.epoch += 1
        if self.buf.is_cuda:
            s = stream if stream is not None else torch.cuda.current_stream(self.buf.device).cuda_stream
            rc = _native.lib().fluxb_barrier_all(
                self._flag_ptrs, self.rank, self.world, ctypes.c_uint32(self.epoch),
                ctypes.c_uint64(int(self.timeout_s * 1e9)), ctypes.c_void_p(self.status.data_ptr()),
                ctypes.c_void_p(s))
            _native.check(rc, "barrier_all")
            return
        for r in range(self.world):
            self._flags[r][self.rank] = self.epoch
        deadline = time.monotonic() + self.timeout_s
        mine = self._flags[self.rank]
        while int(mine.min()) < self.epoch:
            if time.monotonic() > deadline:
                missing = [r for r in range(self.world) if int(mine[r]) < self.epoch]
                raise FluxTimeoutError(f"barrier {self.epoch}: ranks {missing} never arrived")
            time.sleep(0.0002)

    def check(self) -> None:
        """Raise if a device-side wait of an earlier barrier gave up (synchronises)."""
        if self.buf.is_cuda:
            st = self.status.tolist()
            if st[0] != 0:
                raise FluxTimeoutError(f"device barrier timed out: saw {st[2]}, expected {st[3]}")
