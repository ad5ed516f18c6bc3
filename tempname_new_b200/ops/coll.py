"""Stand-alone collectives over symmetric memory: ``AllGatherOp``, ``All2AllSingle``,
``AsyncSendRecv`` (reference: ``src/pybind/flux_coll_op.cc:37-68,352-436``,
``src/coll/ths_op/all_gather_op.cc``, ``src/coll/all2all_impl.cu``, ``src/coll/ths_op/isendrecv.cc``).

One peer-memory kernel (``csrc/ops/a2a.cu``) serves all-gather and variable-split all-to-all; split
sizes are exchanged on the device, so no call synchronises with the host. The ring / copy-engine /
NUMA modes of the reference have no counterpart on an NVSwitch node; their option fields are
accepted and ignored."""
from __future__ import annotations

import ctypes
import time
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native
from . import _dense
from ._fused_base import OFF_CTR, OFF_LOCAL, FusedOpBase
from ..parallel.symm import FluxTimeoutError, SymmBuffer, _ELEM

_VP = ctypes.c_void_p
_R = _dense.MAX_RANKS
_OFF_TABLE = OFF_CTR + 1024      # W*W int32 behind the flags


class A2ARowsArgs(ctypes.Structure):
    _fields_ = [
        ("in_", _VP), ("in_splits", _VP), ("rows_in", ctypes.c_int32), ("broadcast", ctypes.c_int32),
        ("row_bytes", ctypes.c_int64), ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("num_ctas", ctypes.c_int32), ("timeout_ns", ctypes.c_uint64),
        ("status", _VP), ("out", _VP * _R), ("table", _VP * _R), ("flags", _VP * _R), ("local_cnt", _VP),
        ("out_splits", _VP), ("out_offsets", _VP), ("out_capacity_rows", ctypes.c_int64), ("stream", _VP),
    ]


class _RowExchange(FusedOpBase):
    def __init__(self, pg, max_rows: int, n_dim: int, dtype: torch.dtype, timeout_s=None):
        super().__init__(pg, 1, timeout_s)
        self.max_rows, self.n_dim, self.dtype = max_rows, n_dim, dtype
        self.buf = SymmBuffer(max_rows * n_dim * _ELEM[dtype], self.pg)

    def _launch(self, x: torch.Tensor, in_splits: Optional[torch.Tensor], broadcast: bool,
                out_splits: Optional[torch.Tensor], out_offsets: Optional[torch.Tensor], num_ctas: int = 0):
        self._begin_call()
        a = A2ARowsArgs()
        a.in_ = x.data_ptr()
        a.in_splits = in_splits.data_ptr() if in_splits is not None else None
        a.rows_in, a.broadcast = x.shape[0], int(broadcast)
        a.row_bytes = x.shape[1] * x.element_size()
        a.rank, a.world, a.epoch, a.num_ctas = self.rank, self.world, self.epoch, num_ctas
        a.timeout_ns, a.status = int(self.timeout_s * 1e9), self.status.data_ptr()
        for r in range(self.world):
            a.out[r] = self.buf.ptr(r)
            a.flags[r] = self.ctrl.ptr(r, OFF_CTR)
            a.table[r] = self.ctrl.ptr(r, _OFF_TABLE)
        a.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        a.out_splits = out_splits.data_ptr() if out_splits is not None else None
        a.out_offsets = out_offsets.data_ptr() if out_offsets is not None else None
        a.out_capacity_rows = self.max_rows
        a.stream = _dense.current_stream_ptr(x.device)
        _native.check(_native.lib().fluxb_a2a_rows(ctypes.byref(a)), "fluxb_a2a_rows")
        self._after_launch()


class AllGatherOp(_RowExchange):
    """``run(input [M/W, K])`` gathers the shards of all ranks into ``local_input_buffer()``
    ([M, K], symmetric memory); when the call's kernel completes every shard has landed."""

    def __init__(self, tp_group, nnodes: int, max_m_dim: int, k_dim: int, input_dtype: torch.dtype,
                 timeout_s=None):
        super().__init__(tp_group, max_m_dim, k_dim, input_dtype, timeout_s)
        self.k_dim = k_dim
        self._cpu = None
        self._scale_op: Optional[_RowExchange] = None    # built at the first call that carries scales
        self._scales: Optional[torch.Tensor] = None      # [M, 1] fp32 in rank order, of the latest such call

    def _gather_scales(self, input_scale: torch.Tensor, seg: int) -> None:
        """Per-row input scales ([M/W, 1] fp32, the int8 convention of the reference's all-gather op,
        python/flux/cpp_mod.pyi:130-132) travel through a second, small exchange."""
        sc = input_scale.reshape(-1).float().contiguous()
        if sc.numel() != seg:
            raise ValueError(f"input_scale must hold one value per row of the shard ({seg}), got {sc.numel()}")
        if not sc.is_cuda:
            parts = [torch.empty_like(sc) for _ in range(self.world)]
            dist.all_gather(parts, sc, group=self.pg)
            self._scales = torch.cat(parts).reshape(-1, 1)
            return
        rows = (seg + 3) // 4                             # rows of four floats (16 bytes)
        need = (self.max_rows // self.world + 3) // 4 * self.world
        if self._scale_op is None:
            self._scale_op = _RowExchange(self.pg, need, 4, torch.float32, self.timeout_s)
        padded = torch.zeros(rows * 4, dtype=torch.float32, device=sc.device)
        padded[:seg] = sc
        self._scale_op._launch(padded.view(rows, 4), None, True, None, None)
        got = self._scale_op.buf.view(self.rank, torch.float32, (need, 4))[: rows * self.world]
        self._scales = got.reshape(self.world, rows * 4)[:, :seg].reshape(-1, 1).contiguous()

    def run(self, input: torch.Tensor, input_scale=None, all_gather_option=None, stream=None) -> torch.Tensor:
        if input_scale is not None:
            self._gather_scales(input_scale, input.shape[0])
        if not input.is_cuda:
            parts = [torch.empty_like(input) for _ in range(self.world)]
            dist.all_gather(parts, input.contiguous(), group=self.pg)
            self._cpu = torch.cat(parts)
            return self._cpu
        x = input if input.is_contiguous() else input.contiguous()
        self._launch(x, None, True, None, None)
        return self.local_input_buffer()[: x.shape[0] * self.world]

    def local_input_buffer(self) -> torch.Tensor:
        if self._cpu is not None:
            return self._cpu
        return self.buf.view(self.rank, self.dtype, (self.max_rows, self.k_dim))

    def local_barrier_buffer(self) -> torch.Tensor:
        return self.ctrl.view(self.rank, torch.int32, (2 * self.world,), OFF_CTR)

    def local_input_scale_buffer(self) -> Optional[torch.Tensor]:
        """[M, 1] fp32 scales of all ranks' rows, from the latest ``run`` that was given ``input_scale``."""
        return self._scales


class All2AllSingle(_RowExchange):
    """Variable-split all-to-all of rows: ``forward(input [sum(input_splits), n_dim], output,
    input_splits [W], output_splits [W])`` fills ``output`` ordered by source rank and writes the
    received counts into ``output_splits`` (a device int32 tensor)."""

    def __init__(self, pg, max_split: int, n_dim: int, local_world_size: int, input_dtype: torch.dtype,
                 ep_team: int = 0, timeout_s=None):
        world = dist.get_world_size(pg if pg is not None else dist.group.WORLD)
        super().__init__(pg, max_split * world, n_dim, input_dtype, timeout_s)

    def forward(self, input: torch.Tensor, output: Optional[torch.Tensor], input_splits: torch.Tensor,
                output_splits: Optional[torch.Tensor] = None, num_comm_sm: int = 0) -> torch.Tensor:
        if not input.is_cuda:
            ins = [int(v) for v in input_splits.tolist()]
            outs_t = torch.empty(self.world, dtype=torch.int64)
            dist.all_to_all_single(outs_t, torch.tensor(ins, dtype=torch.int64), group=self.pg)
            outs = [int(v) for v in outs_t.tolist()]
            res = torch.empty(sum(outs), input.shape[1], dtype=input.dtype)
            dist.all_to_all_single(res, input.contiguous(), outs, ins, group=self.pg)
            if output_splits is not None:
                output_splits.copy_(outs_t.to(output_splits.dtype))
            if output is not None:
                output[: res.shape[0]].copy_(res)
                return output
            return res
        x = input if input.is_contiguous() else input.contiguous()
        isp = input_splits.to(device=x.device, dtype=torch.int32).contiguous()
        osp = output_splits if (output_splits is not None and output_splits.is_cuda
                                and output_splits.dtype == torch.int32) else \
            torch.empty(self.world, dtype=torch.int32, device=x.device)
        self._launch(x, isp, False, osp, None, num_comm_sm if num_comm_sm > 0 else 0)
        if output_splits is not None and output_splits is not osp:
            output_splits.copy_(osp)
        res = self.buf.view(self.rank, self.dtype, (self.max_rows, self.n_dim))
        if output is not None:
            n = min(output.shape[0], self.max_rows)
            output[:n].copy_(res[:n])
            return output
        return res


All2AllOp = All2AllSingle


class AsyncSendRecv:
    """Host-initiated transfers between symmetric communication buffers with signal words
    (reference: ``flux.AsyncSendRecv``): ``duplicate`` buffers of ``[max_m, n_dim]`` per rank."""

    def __init__(self, max_m: int, n_dim: int, rank: int, world_size: int, input_dtype: torch.dtype,
                 duplicate: int = 1, pg=None):
        self.pg = pg if pg is not None else dist.group.WORLD
        self.rank, self.world = rank, world_size
        self.max_m, self.n_dim, self.dtype, self.dup = max_m, n_dim, input_dtype, duplicate
        self.nbytes = max_m * n_dim * _ELEM[input_dtype]
        self.buf = SymmBuffer(self.nbytes * duplicate, self.pg)
        self.sig = SymmBuffer(256, self.pg)
        self.is_cuda = self.buf.is_cuda

    def get_comm_buffer(self, comm_buff_id: int) -> torch.Tensor:
        return self.buf.view(self.rank, self.dtype, (self.max_m, self.n_dim), comm_buff_id * self.nbytes)

    def _copy(self, dst_ptr: int, src_ptr: int, dst_t: torch.Tensor, src_t: torch.Tensor) -> None:
        if not self.is_cuda:
            dst_t.copy_(src_t)
            return
        rc = _native.lib().fluxb_copy_bytes(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr),
                                            ctypes.c_int64(self.nbytes),
                                            ctypes.c_void_p(_dense.current_stream_ptr(self.buf.device)))
        _native.check(rc, "fluxb_copy_bytes")

    def read_comm_buffer(self, tgt_rank: int, src_comm_buff_id: int, tgt_comm_buff_id: int) -> None:
        """local[src_comm_buff_id] <- tgt_rank's buffer tgt_comm_buff_id"""
        self._copy(self.buf.ptr(self.rank, src_comm_buff_id * self.nbytes),
                   self.buf.ptr(tgt_rank, tgt_comm_buff_id * self.nbytes),
                   self.get_comm_buffer(src_comm_buff_id),
                   self.buf.view(tgt_rank, self.dtype, (self.max_m, self.n_dim), tgt_comm_buff_id * self.nbytes)
                   if not self.is_cuda else None)

    def write_comm_buffer(self, tgt_rank: int, src_comm_buff_id: int, tgt_comm_buff_id: int) -> None:
        """tgt_rank's buffer tgt_comm_buff_id <- local[src_comm_buff_id]"""
        self._copy(self.buf.ptr(tgt_rank, tgt_comm_buff_id * self.nbytes),
                   self.buf.ptr(self.rank, src_comm_buff_id * self.nbytes),
                   self.buf.view(tgt_rank, self.dtype, (self.max_m, self.n_dim), tgt_comm_buff_id * self.nbytes)
                   if not self.is_cuda else None,
                   self.get_comm_buffer(src_comm_buff_id))

    def set_signal(self, tgt_rank: int, comm_buff_id: int, value: int) -> None:
        if not self.is_cuda:
            self.sig.view(tgt_rank, torch.int32, (64,))[comm_buff_id] = value
            return
        rc = _native.lib().fluxb_set_flag(ctypes.c_void_p(self.sig.ptr(tgt_rank, 4 * comm_buff_id)),
                                          ctypes.c_uint32(value),
                                          ctypes.c_void_p(_dense.current_stream_ptr(self.buf.device)))
        _native.check(rc, "fluxb_set_flag")

    def reset_signal(self, comm_buff_id: int) -> None:
        self.set_signal(self.rank, comm_buff_id, 0)

    def wait_signal_eq(self, comm_buff_id: int, value: int, timeout_s: float = 10.0) -> None:
        """Waits (stream-ordered on CUDA, bounded) until the local signal equals ``value``. On CUDA
        the wait is a kernel on the current stream: if it runs out of time the stream goes on and
        the outcome is in the op's status word, which ``check()`` (or the next ``wait_signal_eq``)
        turns into ``FluxTimeoutError``."""
        if not self.is_cuda:
            w = self.sig.view(self.rank, torch.int32, (64,))
            deadline = time.monotonic() + timeout_s
            while int(w[comm_buff_id]) != value:
                if time.monotonic() > deadline:
                    raise FluxTimeoutError(f"signal {comm_buff_id} never became {value}")
                time.sleep(0.0002)
            return
        if not hasattr(self, "_status"):
            self._status = torch.zeros(4, dtype=torch.int32, device=self.buf.device)
            self._waits_unchecked = 0
        elif self._waits_unchecked >= 64:
            self.check()       # an earlier wait may have given up: do not pile more work on top of it
        rc = _native.lib().fluxb_wait_flag_eq(ctypes.c_void_p(self.sig.ptr(self.rank, 4 * comm_buff_id)),
                                              ctypes.c_uint32(value), ctypes.c_uint64(int(timeout_s * 1e9)),
                                              ctypes.c_void_p(self._status.data_ptr()),
                                              ctypes.c_void_p(_dense.current_stream_ptr(self.buf.device)))
        _native.check(rc, "fluxb_wait_flag_eq")
        self._waits_unchecked += 1

    def check(self) -> None:
        """Synchronise and raise ``FluxTimeoutError`` if a signal wait since the last check gave up
        (the consumers of the comm buffer then ran on data that never arrived)."""
        if not self.is_cuda or not hasattr(self, "_status"):
            return
        st = self._status.tolist()
        self._waits_unchecked = 0
        if st[0] != 0:
            self._status.zero_()
            raise FluxTimeoutError(f"AsyncSendRecv: a signal wait timed out (saw {st[2] & 0xFFFFFFFF}, "
                                   f"waited for {st[3] & 0xFFFFFFFF})")
