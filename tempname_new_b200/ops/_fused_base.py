"""State shared by the fused dense ops: the per-op control block in symmetric memory (start
flags, arrival counters), the call counter ("epoch") that replaces per-call flag resets, and
the device status word that bounded waits report into."""
from __future__ import annotations

import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.symm import FluxTimeoutError, SymmBuffer

# byte offsets inside the control block
OFF_START = 0          # [8] uint32  last call number entered, by source rank
OFF_WORK = 64          # [1] uint32  this op's wave counter (tile starts kept in step, zero between calls)
OFF_CTR = 128          # arrival flags written by peers, op specific (up to 32 KiB)
OFF_LOCAL = 32 * 1024  # local arrival scratch (never touched by peers)
CTRL_BYTES = 64 * 1024
MAX_FLAG_WORDS = (OFF_LOCAL - OFF_CTR) // 4

SITE_NAMES = {
    1: "smem-empty barrier", 2: "smem-full barrier", 3: "tmem-empty barrier", 4: "tmem-full barrier",
    5: "start handshake", 6: "all-gather shard flag", 7: "reduce-scatter tile counter",
    8: "barrier_all", 9: "inplace cast", 10: "all-to-all flag", 11: "MoE flag", 12: "test wait",
    13: "receive buffer capacity (rows routed to one rank)",
}
# self-checks of the debug build (FLUXB_DEBUG=1), csrc/sm100/ptx.cuh::CheckSite
CHECK_NAMES = {
    101: "tile coordinates outside the problem", 102: "all-gather push outside the shard or misaligned",
    103: "post-attention push outside its buffers", 104: "MoE gather index outside the token matrix",
    105: "flag carries a call number far ahead of the current call", 106: "epilogue store outside the output",
}


class FluxDeviceCheckError(RuntimeError):
    """A device-side self-check of the debug build failed."""


class FusedOpBase:
    def __init__(self, pg, nnodes: int = 1, timeout_s: Optional[float] = None):
        if nnodes != 1:
            raise NotImplementedError(
                "multi-node operation is outside the single NVSwitch domain this library targets")
        self.pg = pg if pg is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.pg)
        self.world = dist.get_world_size(self.pg)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVSwitch node)")
        self.epoch = 0
        env_t = os.environ.get("FLUXB_WAIT_TIMEOUT_S")
        self.timeout_s = timeout_s if timeout_s is not None else (float(env_t) if env_t else 5.0)
        self.ctrl = SymmBuffer(CTRL_BYTES, self.pg)
        self.is_cuda = self.ctrl.is_cuda
        self.device = self.ctrl.device
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device) if self.is_cuda else None
        self.check_every_call = os.environ.get("FLUXB_CHECK_STATUS", "0") == "1"
        # set when a wait of this op gave up: its arrival counters may be left partly counted and
        # the ranks' call numbers may disagree, so the op refuses to run until reset()
        self.poisoned: Optional[str] = None
        # SMs left free for other work (a collective of another group, a second stream): the fused
        # kernels keep all their CTAs resident and wait for one another, so they must not be launched
        # wider than what is free. Per-call ``sm_margin`` arguments override this default
        # (reference: ``sm_margin`` / ``num_comm_sm`` of the Ulysses and MoE ops, e.g.
        # src/gemm_a2a_transpose/ths_op/gemm_all2all_transpose.cc:559-560).
        self.sm_margin = int(os.environ.get("FLUXB_SM_MARGIN", "0"))
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count if self.is_cuda else 0

    # -- device status ---------------------------------------------------------------
    def check_status(self) -> None:
        """Synchronise and raise FluxTimeoutError if a device wait of this op gave up."""
        if self.status is None:
            return
        st = self.status.tolist()
        if st[0] >= 100:
            self.status.zero_()
            self.poisoned = "a device-side check failed"
            raise FluxDeviceCheckError(
                f"{type(self).__name__}: device check '{CHECK_NAMES.get(st[0], st[0])}' failed in block {st[1]} "
                f"(details {st[2] & 0xFFFFFFFF}, {st[3] & 0xFFFFFFFF})")
        if st[0] != 0:
            self.status.zero_()
            self.poisoned = "a device wait timed out"
            raise FluxTimeoutError(
                f"{type(self).__name__}: device wait '{SITE_NAMES.get(st[0], st[0])}' timed out in "
                f"block {st[1]} (saw {st[2] & 0xFFFFFFFF}, expected {st[3] & 0xFFFFFFFF})")

    def _after_launch(self) -> None:
        if self.check_every_call:
            self.check_status()

    def _num_sms(self, sm_margin: Optional[int] = None) -> int:
        """SMs a launch of this op may use: 0 (= all) without a margin, else the device's count minus
        the margin (at least 2)."""
        m = self.sm_margin if not sm_margin else sm_margin
        if m <= 0 or self._sm_count == 0:
            return 0
        return max(self._sm_count - m, 2)

    def _begin_call(self) -> int:
        """Every forward starts here: refuses a poisoned op, then takes the next call number."""
        if self.poisoned is not None:
            raise RuntimeError(
                f"{type(self).__name__}: {self.poisoned} in an earlier call; its counters and the ranks' call "
                "numbers may be inconsistent. Call reset() on every rank of the group before using it again.")
        self.epoch += 1
        return self.epoch

    # -- recovery ----------------------------------------------------------------------
    def _local_scratch_regions(self):
        """(offset, bytes) ranges of the control block that only this rank's kernels write and
        that must read zero between calls: the work-claim word and the arrival scratch."""
        return [(OFF_WORK, 64), (OFF_LOCAL, CTRL_BYTES - OFF_LOCAL)]

    def reset(self) -> None:
        """Collective over the op's group: bring the op back to a usable state after a
        ``FluxTimeoutError`` / ``FluxDeviceCheckError`` (or any failed call). Waits for this
        rank's outstanding work, zeroes the local arrival counters that an aborted kernel may
        have left partly counted (and the launcher's wave counters), agrees on a call number
        above every rank's, and clears the status word. Flags written by peers need no clearing:
        they carry call numbers, and the agreed number is larger than any of them."""
        if self.is_cuda:
            torch.cuda.synchronize(self.device)
        for off, nbytes in self._local_scratch_regions():
            self.ctrl.local[off:off + nbytes].zero_()
        if self.is_cuda:
            from .. import _native
            _native.check(_native.lib().fluxb_reset_wave_counters(), "fluxb_reset_wave_counters")
            self.status.zero_()
            torch.cuda.synchronize(self.device)
        t = torch.tensor([self.epoch], dtype=torch.int64, device=self.device if self.is_cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        self.epoch = int(t.item()) + 1     # the next call uses a number no rank has used
        self.poisoned = None
        dist.barrier(group=self.pg)

    # -- CPU emulation of the flag protocol -------------------------------------------
    def _cpu_words(self, r: int, off: int, n: int) -> torch.Tensor:
        return self.ctrl.view(r, torch.int32, (n,), off)

    def _cpu_wait(self, words: torch.Tensor, expected: int, what: str) -> None:
        deadline = time.monotonic() + self.timeout_s
        while int(words.min()) < expected:
            if time.monotonic() > deadline:
                late = [i for i in range(words.numel()) if int(words[i]) < expected]
                self.poisoned = f"the wait for {what} timed out"
                raise FluxTimeoutError(f"{type(self).__name__}: {what} timed out waiting for {late}")
            time.sleep(0.0002)

    def _cpu_start_handshake(self) -> None:
        for r in range(self.world):
            self._cpu_words(r, OFF_START, 8)[self.rank] = self.epoch
        self._cpu_wait(self._cpu_words(self.rank, OFF_START, 8)[: self.world], self.epoch, "start handshake")
