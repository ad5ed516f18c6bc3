"""``GemmRS``: GEMM fused with reduce-scatter (row-parallel linear forward).

``out[M/W, N] = reduce_scatter_M(input[M, K/W] @ weight[N, K/W]^T (+bias))``

On CUDA one persistent tcgen05 kernel does everything: each output tile of M-segment ``s``
leaves the epilogue as a TMA store straight into rank ``s``'s staging slab ``[this rank]``
over NVLink, segments are visited ``rank+1, rank+2, …, rank`` so that every step is a
permutation on the switch, an arrival counter per tile row is bumped once the store has
landed, and the tail of the same kernel sums the ``W`` slabs in fp32 in a fixed order.
Reference: ``flux.GemmRS`` (``src/pybind/gemm_rs.cc:28-92``,
``src/gemm_rs/ths_op/gemm_reduce_scatter.cc``); there the sm90 path pulls tiles with TMA into
a ``[W, M/W, N]`` buffer and a separate kernel reduces it.
"""
from __future__ import annotations

import dataclasses

from typing import Optional

import torch
import torch.distributed as dist

from . import _dense
from ._fused_base import MAX_FLAG_WORDS, OFF_CTR, OFF_LOCAL, OFF_START, OFF_WORK, FusedOpBase
from .gemm_only import _out_dtype, as_nk
from .options import ReduceScatterOption
from ..parallel.symm import SymmBuffer, _ELEM


class GemmRS(FusedOpBase):
    def __init__(self, tp_group, nnodes: int, max_m: int, n_dim: int, input_dtype: torch.dtype,
                 output_dtype: Optional[torch.dtype] = None, transpose_weight: bool = False,
                 fuse_reduction: bool = False, ring_reduction: bool = False,
                 timeout_s: Optional[float] = None):
        super().__init__(tp_group, nnodes, timeout_s)
        self.max_m, self.n_dim = max_m, n_dim
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.transpose_weight = transpose_weight
        self.fuse_reduction = fuse_reduction      # accepted; the reduction is always fused in-kernel
        self.ring_reduction = ring_reduction      # accepted; the sum order is fixed (rank 0..W-1)
        if max_m % self.world != 0:
            raise ValueError("max_m must be a multiple of the world size")
        if (max_m // self.world + 127) // 128 * 8 > MAX_FLAG_WORDS:
            raise ValueError("max_m too large for the flag block")
        # staging: W slabs of [max_m / W, N] on every rank
        self.stage = SymmBuffer(max_m * n_dim * _ELEM[self.output_dtype], self.pg) if self.world > 1 else None

    def zero_buffers(self) -> None:
        """Kept for API compatibility: counters carry the call number, nothing needs zeroing."""

    # ------------------------------------------------------------------------------------
    def forward(self, input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                input_scale: Optional[torch.Tensor] = None, weight_scale: Optional[torch.Tensor] = None,
                output_scale: Optional[torch.Tensor] = None, fast_accum: bool = False,
                reduce_scatter_option: Optional[ReduceScatterOption] = None,
                transpose_weight_override: Optional[bool] = None) -> torch.Tensor:
        tw = self.transpose_weight if transpose_weight_override is None else transpose_weight_override
        w = as_nk(weight, tw)
        M, N = input.shape[0], w.shape[0]
        if M > self.max_m or N != self.n_dim:
            raise ValueError(f"GemmRS was built for M <= {self.max_m}, N = {self.n_dim}; got M={M}, N={N}")
        if M % self.world != 0:
            raise ValueError("M must be a multiple of the world size")
        self._begin_call()
        if not input.is_cuda:
            return self._forward_cpu(input, w, bias, input_scale, weight_scale)
        a = input if input.stride(-1) == 1 else input.contiguous()
        out = torch.empty((M // self.world, N), dtype=self.output_dtype, device=input.device)
        keep: list = []
        if input_scale is not None and input_scale.dim() == 3:
            from .blockscale_gemm import blockscale_args
            if (M // self.world) % 128:
                raise ValueError("block-scaled GEMM+RS needs M/W to be a multiple of 128")
            args = blockscale_args(a, w, input_scale, weight_scale, bias, self.output_dtype, M,
                                   status=self.status, keep=keep)
        else:
            args = _dense.base_args(a, w, bias, self.output_dtype, input_scale, weight_scale,
                                    m=M, status=self.status, keep=keep)
        args.M = M
        args.num_sms = self._num_sms()
        args.mode, args.rank, args.world = _dense.REDUCE_SCATTER, self.rank, self.world
        args.epoch = self.epoch
        args.timeout_ns = int(self.timeout_s * 1e9)
        args.rs_out = out.data_ptr()
        if self.world > 1:
            for r in range(self.world):
                args.rs_stage[r] = self.stage.ptr(r)
                args.rs_ctr[r] = self.ctrl.ptr(r, OFF_CTR)
                args.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
            args.wave_ctr = self.ctrl.ptr(self.rank, OFF_WORK)
            args.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        _dense.run(args)
        self._after_launch()
        return out

    __call__ = forward

    def forward_barrier(self, input, weight, bias=None):
        """Reference API: the barrier between GEMM and reduction. The fused kernel needs none."""

    def forward_reduce_scatter(self, input, weight, bias=None, input_scale=None, weight_scale=None):
        return self.forward(input, weight, bias, input_scale, weight_scale)

    def profiling(self, input, weight, bias=None, input_scale=None, weight_scale=None, output_scale=None,
                  fast_accum=False, reduce_scatter_option=None, prof_ctx=None):
        from ..tuning.profiling import profile_call
        w = as_nk(weight, self.transpose_weight)
        blockscaled = input_scale is not None and input_scale.dim() == 3
        key = None if blockscaled else (input.shape[0], w.shape[0], input.shape[1])
        return profile_call(self, "gemm_rs", lambda: self.forward(input, weight, bias, input_scale, weight_scale),
                            prof_ctx, key=key, segmented_rows=input.shape[0] // self.world)

    # ------------------------------------------------------------------------------------
    def _forward_cpu(self, a, w, bias, sa, sb):
        """Same data movement on shared host memory: push each partial segment into the owner's
        slab, signal, then the owner sums its W slabs in rank order."""
        W, r = self.world, self.rank
        M, N = a.shape[0], w.shape[0]
        seg = M // W
        part = a.float() @ w.float().t()
        if sa is not None:
            vec = _dense.check_scale(sa, a.shape[0], "input_scale")
            part = part * (sa.float().reshape(-1, 1) if vec else sa.float().reshape(-1)[0])
        if sb is not None:
            vec = _dense.check_scale(sb, w.shape[0], "weight_scale")
            part = part * (sb.float().reshape(1, -1) if vec else sb.float().reshape(-1)[0])
        if bias is not None:
            part = part + bias.float()
        part = part.to(self.output_dtype)
        if W == 1:
            return part
        self._cpu_start_handshake()
        for d in range(1, W + 1):
            s = (r + d) % W
            slab = self.stage.view(s, self.output_dtype, (W, seg, N))
            slab[r].copy_(part[s * seg:(s + 1) * seg])
            self._cpu_words(s, OFF_CTR, 8)[r] = self.epoch
        self._cpu_wait(self._cpu_words(r, OFF_CTR, 8)[:W], self.epoch, "reduce-scatter arrivals")
        mine = self.stage.view(r, self.output_dtype, (W, seg, N))
        return mine.float().sum(0).to(self.output_dtype)


@dataclasses.dataclass
class SegmentInfo:
    """One run of consecutive tile rows that keeps its order when the GEMM re-orders its tile
    rows for the reduce-scatter (reference: ``SegmentInfo``, src/pybind/gemm_rs.cc:104-108)."""
    segment_origin: int        # owner rank of the rows
    size: int                  # tile rows in the run
    tile_m_start_origin: int   # first tile row in the output's own order
    tile_m_start_new: int      # first tile row in the order the kernel visits them


def get_gemm_rs_threadblock_segments_info(problem_shape, tiled_shape, rank: int, world_size: int,
                                          sub_world_size: int = 0, nnodes: int = 1, use_2d_ring: bool = False,
                                          per_tile_flags: bool = False):
    """The order in which the reduce-scatter GEMM of this library visits the output: the segment
    of rank+1 first, its own segment last, so that every owner receives its partial tiles spread
    over the whole run and computes its own contribution when the others have arrived. The
    reference computes the analogous table for its PCIe / 2-D ring orders
    (src/pybind/gemm_rs.cc:110-140, ``ThreadBlockSwizzleSegmentUtils``); ``sub_world_size``,
    ``use_2d_ring`` and ``per_tile_flags`` select orders that one NVSwitch domain does not need."""
    if nnodes != 1:
        raise NotImplementedError("one NVSwitch node")
    M, tile_m = int(problem_shape[0]), int(tiled_shape[0])
    if M % world_size:
        raise ValueError("M must divide over the ranks")
    per_seg = -(-(M // world_size) // tile_m)
    out = []
    for i in range(world_size):
        seg = (rank + 1 + i) % world_size
        out.append(SegmentInfo(seg, per_seg, seg * per_seg, i * per_seg))
    return out


def calc_gemm_rs_threadblock_segments_info(segments: torch.Tensor, problem_shape, tiled_shape, rank: int,
                                           world_size: int, sub_world_size: int = 0, nnodes: int = 1,
                                           use_2d_ring: bool = False, per_tile_flags: bool = False) -> int:
    """Writes the table above into ``segments`` ([>= world_size, 4] int32) and returns its length."""
    info = get_gemm_rs_threadblock_segments_info(problem_shape, tiled_shape, rank, world_size, sub_world_size,
                                                 nnodes, use_2d_ring, per_tile_flags)
    flat = segments.view(-1, 4)
    for i, s in enumerate(info):
        flat[i] = torch.tensor([s.segment_origin, s.size, s.tile_m_start_origin, s.tile_m_start_new],
                               dtype=flat.dtype)
    return len(info)

