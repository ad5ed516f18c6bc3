"""Expert-parallel token dispatch / combine and the remaining transport helpers, single node.

* ``DisScatterForward``: every rank contributes its local tokens; each rank receives, in
  expert-sorted order, the rows routed to its own experts (reference: ``flux.DisScatterForward``,
  ``src/coll/dis_scatter_forward_impl.cu``; there a hierarchical NVSHMEM put/signal protocol that
  also spans nodes). Here one kernel (``csrc/ops/ep_dispatch.cu``) stores every routed row
  straight into its place in the receiver's buffer over NVLink: a token travels only to the ranks
  that own one of its experts.
* ``DisScatterBackward``: the inverse, the weighted combine: the expert outputs of all ranks are
  summed per token over the top-k entries and delivered to the rank that owns the token — the
  ``moe_combine_kernel`` used by ``GemmGroupedV3GatherRS`` (reference:
  ``src/coll/dis_scatter_backward_impl.cu``).
* ``All2AllInference``, ``TransportOp``: thin wrappers over the row-exchange and copy kernels.
* ``GemmRSInterNode`` / ``GemmRS_multinode`` / ``AGKernelInterNode`` / ``AGKernelXNode``: multi-node
  variants; this library targets one NVSwitch domain, so constructing them raises.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from . import _dense
from ._fused_base import OFF_CTR, OFF_LOCAL, OFF_START, FusedOpBase
from .coll import All2AllSingle, AllGatherOp
from .moe import GemmGroupedV3GatherRS, _scratch
from ..parallel.symm import SymmBuffer, _ELEM

_VP = ctypes.c_void_p
_R = _dense.MAX_RANKS


class EpDispatchArgs(ctypes.Structure):
    _fields_ = [
        ("x", _VP), ("scatter_index", _VP), ("splits", _VP), ("token0", ctypes.c_int64),
        ("tokens_local", ctypes.c_int32), ("topk", ctypes.c_int32), ("E", ctypes.c_int32),
        ("E_local", ctypes.c_int32), ("tp", ctypes.c_int32), ("num_ctas", ctypes.c_int32),
        ("row_bytes", ctypes.c_int64), ("capacity_rows", ctypes.c_int64),
        ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64), ("status", _VP),
        ("out", _VP * _R), ("flags", _VP * _R), ("start_ctr", _VP * _R),
        ("local_cnt", _VP), ("out_rows", _VP), ("stream", _VP),
    ]


class DisScatterForward(FusedOpBase):
    def __init__(self, total_num_experts: int, max_m: int, n_dim: int, topk: int, rank: int, tp_world_size: int,
                 ep_world_size: int, local_world_size: int, moe_capacity_ratio: float = 1.3,
                 duplicate_comm_buffer: int = 1, team: int = 0, pg=None, dtype: torch.dtype = torch.bfloat16,
                 timeout_s: Optional[float] = None):
        super().__init__(pg, 1, timeout_s)
        if rank != self.rank:
            raise ValueError("rank must be this process's rank in the group")
        if tp_world_size * ep_world_size != self.world:
            raise ValueError("tp_world_size * ep_world_size must equal the group size")
        self.E, self.topk, self.H = total_num_experts, topk, n_dim
        self.tp = tp_world_size
        self.E_local = self.E // ep_world_size
        self.e0 = (rank // tp_world_size) * self.E_local
        self.dtype = dtype
        self.max_m = max_m
        self._index_ag = {}
        if self.is_cuda:
            # rows one rank can receive: its fair share of max_m * topk times the capacity ratio
            total = max(max_m * topk, 1)
            self.capacity = min(total, int(math.ceil(total / ep_world_size * moe_capacity_ratio)))
            self.recv = SymmBuffer(self.capacity * n_dim * _ELEM[dtype], self.pg)
            self.ag = None
        else:
            self.ag = AllGatherOp(self.pg, 1, max_m, n_dim, dtype)

    def _token0(self, tokens_local: int, ep_token_counts) -> int:
        if ep_token_counts is None:
            return self.rank * tokens_local
        counts = ep_token_counts.tolist() if torch.is_tensor(ep_token_counts) else list(ep_token_counts)
        return int(sum(counts[: self.rank]))

    def forward_gpu(self, input: torch.Tensor, ag_exp_indices: torch.Tensor, ag_scatter_idx: torch.Tensor,
                    splits: torch.Tensor, ep_token_counts=None, output_tensor: Optional[torch.Tensor] = None,
                    sm_margin: int = 0, copy_to_local_tensor: bool = True) -> torch.Tensor:
        """input [local tokens, H]; ag_scatter_idx [tokens, topk] = sorted row of every (token, k);
        splits [E] rows per expert. Returns this rank's rows [sum(splits[e0:e0+E_local]), H]
        (``copy_to_local_tensor=False``: a view of the receive buffer, valid until the next call)."""
        if input.is_cuda:
            return self._forward_cuda(input, ag_scatter_idx, splits, ep_token_counts, output_tensor,
                                      copy_to_local_tensor)
        tokens_full = self.ag.run(input)
        n = ag_scatter_idx.numel()
        topk = ag_scatter_idx.shape[-1]
        gather = torch.empty(n, dtype=torch.long, device=input.device)
        gather[ag_scatter_idx.reshape(-1).long()] = torch.arange(n, device=input.device) // topk
        offs = torch.cat([torch.zeros(1, dtype=torch.long, device=splits.device), splits.long().cumsum(0)])
        lo, hi = int(offs[self.e0]), int(offs[self.e0 + self.E_local])
        out = tokens_full.index_select(0, gather[lo:hi])
        if output_tensor is not None:
            output_tensor[: out.shape[0]].copy_(out)
            return output_tensor
        return out

    def _forward_cuda(self, x, scatter_idx, splits, ep_token_counts, output_tensor, copy_out) -> torch.Tensor:
        dev = x.device
        x = x if x.is_contiguous() else x.contiguous()
        if x.dtype != self.dtype or x.shape[1] != self.H:
            raise ValueError("input must be [tokens, n_dim] in the dtype the op was built for")
        sidx = scatter_idx.reshape(-1).to(device=dev, dtype=torch.int32).contiguous()
        # the row count of this rank comes from the host copy of the splits when there is one
        sp_host = splits if not splits.is_cuda else None
        sp = splits.to(device=dev, dtype=torch.int32, non_blocking=True).contiguous()
        self._begin_call()
        a = EpDispatchArgs()
        a.x, a.scatter_index, a.splits = x.data_ptr(), sidx.data_ptr(), sp.data_ptr()
        a.tokens_local, a.topk, a.E, a.E_local, a.tp = x.shape[0], self.topk, self.E, self.E_local, self.tp
        a.token0 = self._token0(x.shape[0], ep_token_counts)
        a.row_bytes = self.H * x.element_size()
        a.capacity_rows = self.capacity
        a.rank, a.world, a.epoch = self.rank, self.world, self.epoch
        a.timeout_ns, a.status = int(self.timeout_s * 1e9), self.status.data_ptr()
        for r in range(self.world):
            a.out[r] = self.recv.ptr(r)
            a.flags[r] = self.ctrl.ptr(r, OFF_CTR)
            a.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
        a.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        a.stream = _dense.current_stream_ptr(dev)
        _native.check(_native.lib().fluxb_ep_dispatch(ctypes.byref(a)), "fluxb_ep_dispatch")
        self._after_launch()
        if sp_host is None:
            sp_host = splits.cpu()
        rows = int(sp_host[self.e0:self.e0 + self.E_local].sum())
        if rows > self.capacity:
            self.check_status()
        view = self.recv.view(self.rank, self.dtype, (self.capacity, self.H))[:rows]
        if output_tensor is not None:
            output_tensor[:rows].copy_(view)
            return output_tensor
        return view.clone() if copy_out else view

    def forward(self, input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts=None, sm_margin: int = 0,
                copy_to_local_tensor: bool = True):
        sp = splits_cpu if input.is_cuda else splits_cpu.to(input.device)
        return self.forward_gpu(input, ag_exp_indices, ag_scatter_idx, sp, ep_token_counts, None, sm_margin,
                                copy_to_local_tensor)

    def forward_no_cpy(self, input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts=None,
                       sm_margin: int = 0):
        return self.forward(input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts, sm_margin, False)

    def forward_gpu_no_cpy(self, input, ag_exp_indices, ag_scatter_idx, splits, ep_token_counts=None,
                           output_tensor=None, sm_margin: int = 0):
        return self.forward_gpu(input, ag_exp_indices, ag_scatter_idx, splits, ep_token_counts, output_tensor,
                                sm_margin, False)

    def pre_comm_index(self, ep_token_counts: torch.Tensor, cur_topk_indices: torch.Tensor,
                       cur_topk_values: torch.Tensor, ag_topk_indices: torch.Tensor, ag_topk_values: torch.Tensor,
                       sm_margin: int = 0) -> None:
        """Gather every rank's routing choice ([tokens_r, topk] expert ids and gate values,
        ``ep_token_counts[r]`` tokens on rank r) into the two outputs, rank after rank (reference:
        ``DisScatterForward.pre_comm_index``, python/flux/cpp_mod.pyi:1169-1177)."""
        if cur_topk_indices.is_cuda:
            # rows of bytes through the row-exchange kernel (variable rows per rank, ordered by source);
            # nothing visits the host
            for which, (cur, out) in enumerate(((cur_topk_indices, ag_topk_indices),
                                                (cur_topk_values, ag_topk_values))):
                row_b = cur.shape[1] * cur.element_size()
                pad_b = (row_b + 15) // 16 * 16
                rows = cur.contiguous().view(torch.uint8).reshape(cur.shape[0], row_b)
                if pad_b != row_b:
                    rows = torch.nn.functional.pad(rows, (0, pad_b - row_b))
                key = (which, pad_b)
                if key not in self._index_ag:
                    self._index_ag[key] = AllGatherOp(self.pg, 1, self.max_m, pad_b, torch.uint8)
                ag = self._index_ag[key]
                ag.run(rows.contiguous())
                got = ag.local_input_buffer()[: out.shape[0]]   # rows of all ranks, ordered by source
                out.copy_(got[:, :row_b].contiguous().view(cur.dtype).reshape(out.shape))
            return
        counts = [int(v) for v in ep_token_counts.tolist()]
        mx = max(counts)
        for cur, out in ((cur_topk_indices, ag_topk_indices), (cur_topk_values, ag_topk_values)):
            pad = torch.zeros((mx,) + tuple(cur.shape[1:]), dtype=cur.dtype, device=cur.device)
            pad[: cur.shape[0]] = cur
            parts = [torch.empty_like(pad) for _ in range(self.world)]
            dist.all_gather(parts, pad, group=self.pg)
            row = 0
            for r, n in enumerate(counts):
                out[row:row + n] = parts[r][:n]
                row += n

    def profiling(self, input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts=None, sm_margin: int = 0,
                  copy_to_local_tensor: bool = True, prof_ctx=None):
        from ..tuning.profiling import profile_call
        return profile_call(self, "dis_scatter_forward",
                            lambda: self.forward(input, ag_exp_indices, ag_scatter_idx, splits_cpu), prof_ctx)

    def ep_barrier_all(self) -> None:
        dist.barrier(group=self.pg)


class DisScatterBackward:
    def __init__(self, total_num_experts: int, max_m: int, n_dim: int, topk: int, rank: int, tp_world_size: int,
                 ep_world_size: int, local_world_size: int, moe_capacity_ratio: float = 1.3,
                 duplicate_comm_buffer: int = 1, team: int = 0, pg=None, dtype: torch.dtype = torch.bfloat16):
        self.pg = pg if pg is not None else dist.group.WORLD
        world = dist.get_world_size(self.pg)
        self.op = GemmGroupedV3GatherRS(total_num_experts, max_m * topk if max_m * topk else topk, n_dim, topk, rank,
                                        world, tp_world_size, ep_world_size, tp_group=self.pg, dtype=dtype)

    def forward_gpu(self, input: torch.Tensor, ag_exp_indices, ag_scatter_idx: torch.Tensor, splits: torch.Tensor,
                    ep_token_counts=None, output_tensor: Optional[torch.Tensor] = None, sm_margin: int = 0,
                    copy_to_local_tensor: bool = True) -> torch.Tensor:
        """input [rows of this rank's experts, H] (already gate-weighted) -> [local tokens, H]:
        per token the sum of its top-k rows over all ranks."""
        op = self.op
        ridx = ag_scatter_idx.reshape(-1)
        tokens = ridx.numel() // op.topk
        tpr = tokens // op.world
        if not input.is_cuda:
            offs = torch.cat([torch.zeros(1, dtype=torch.long), splits.long().cumsum(0)])
            base = int(offs[op.e0])
            full = torch.zeros(tokens, input.shape[1])
            r = ridx.reshape(tokens, op.topk).long() - base
            ok = (r >= 0) & (r < input.shape[0])
            for k in range(op.topk):
                sel = ok[:, k]
                full[sel] += input[r[sel, k]].float()
            out = torch.empty(tpr, input.shape[1], dtype=input.dtype)
            dist.reduce_scatter(out, [c.contiguous() for c in full.to(input.dtype).chunk(op.world)], group=self.pg)
        else:
            dev = input.device
            if op._scratch is None:
                op._scratch = _scratch(op.E, op.world, dev)
            # the combine kernel reads (row_base, rows) from the schedule header: fill it here
            offs = torch.cat([torch.zeros(1, dtype=torch.int32, device=dev),
                              splits.to(dev).to(torch.int32).cumsum(0).to(torch.int32)])
            lib = _native.lib()
            lib.fluxb_moe_hdr_offset.restype = ctypes.c_int64
            hdr_off = int(lib.fluxb_moe_hdr_offset(op.E, op.world))
            hdr = op._scratch[hdr_off:hdr_off + 8].view(torch.int32)
            hdr[0] = offs[op.e0]
            hdr[1] = offs[op.e0 + op.E_local] - offs[op.e0]
            out = torch.empty((tpr, input.shape[1]), dtype=input.dtype, device=dev)
            op._combine(input.contiguous(), ridx.to(device=dev, dtype=torch.int32).contiguous(), tpr, out)
        if output_tensor is not None:
            output_tensor[: out.shape[0]].copy_(out)
            return output_tensor
        return out

    def forward(self, input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts=None, sm_margin: int = 0,
                copy_to_local_tensor: bool = True):
        return self.forward_gpu(input, ag_exp_indices, ag_scatter_idx, splits_cpu, ep_token_counts, None, sm_margin)

    forward_no_cpy = forward
    forward_gpu_no_cpy = forward_gpu

    def ep_barrier_all(self) -> None:
        dist.barrier(group=self.pg)

    local_barrier_all = ep_barrier_all


class TopkReduceScatterOp:
    """The communication half of MoE layer 1 on its own: expert outputs (already computed, one
    tensor per weight group) -> per token the gate-weighted sum of its top-k rows over all ranks,
    delivered to the token's owner (reference: ``TopkReduceScatterOp``,
    src/pybind/gemm_grouped_v2_gather_rs.cc:166-215, src/moe_gather_rs/topk_gather_rs.cu). Runs on
    ``moe_combine_kernel``; ``barriers``, ``n_split`` and ``use_read_mode`` select protocols that do
    not exist here and are accepted for signature compatibility."""

    def __init__(self, tp_group, max_m: int, n_dim: int, topk: int, output_dtype: torch.dtype,
                 num_experts: int, ep_world_size: int, barriers=None, n_split: int = 4,
                 do_all_reduce: bool = False, use_read_mode: bool = False):
        self.pg = tp_group if tp_group is not None else dist.group.WORLD
        world, rank = dist.get_world_size(self.pg), dist.get_rank(self.pg)
        if world % ep_world_size:
            raise ValueError("ep_world_size must divide the group")
        self.do_all_reduce = do_all_reduce
        self.inner = DisScatterBackward(num_experts, max_m // max(topk, 1), n_dim, topk, rank, world // ep_world_size,
                                        ep_world_size, world, pg=self.pg, dtype=output_dtype)

    def run(self, gemm_outs, output: Optional[torch.Tensor], ep_start: int, ep_nexperts: int, splits: torch.Tensor,
            routing_idx: torch.Tensor, output_vec_scales=None, num_thread_blocks: int = 0, stream=None) -> torch.Tensor:
        op = self.inner.op
        if ep_start != op.e0 or ep_nexperts != op.E_local:
            raise ValueError("ep_start / ep_nexperts must describe this rank's experts")
        y = None
        for g, t in enumerate(gemm_outs):
            part = t
            if output_vec_scales is not None and output_vec_scales[g] is not None:
                part = (t.float() * output_vec_scales[g].float().reshape(-1, 1)).to(t.dtype)
            y = part if y is None else y + part
        out = self.inner.forward_gpu(y, None, routing_idx, splits)
        if self.do_all_reduce:
            parts = [torch.empty_like(out) for _ in range(op.world)]
            dist.all_gather(parts, out, group=self.pg)
            out = torch.cat(parts)
        if output is not None:
            output[: out.shape[0]].copy_(out)
            return output
        return out

    def reset_buffer(self) -> None:
        """Nothing to reset: flags carry the call number."""


class All2AllInference:
    """Token all-to-all for inference-time EP (reference: ``flux.All2AllInference``): the caller
    fills ``get_input_buffer`` and gives the cumulative row splits per destination."""

    def __init__(self, max_m: int, n_dim: int, rank: int, total_num_experts: int, world_size: int,
                 local_world_size: int, max_element_size: int, pg=None):
        self.pg = pg if pg is not None else dist.group.WORLD
        self.world, self.rank, self.n_dim, self.max_m = world_size, rank, n_dim, max_m
        self._ops = {}
        self._inputs = {}

    def _dtype(self, element_size: int) -> torch.dtype:
        return {1: torch.uint8, 2: torch.bfloat16, 4: torch.float32}[element_size]

    def get_input_buffer(self, input_shape, element_size: int, with_scale: bool = False) -> torch.Tensor:
        dt = self._dtype(element_size)
        dev = "cuda" if torch.cuda.is_available() and "nccl" in str(dist.get_backend(self.pg)) else "cpu"
        buf = torch.empty(tuple(input_shape), dtype=dt, device=dev)
        self._inputs[element_size] = buf
        return buf

    def forward(self, input_size, input_split_cumsum: torch.Tensor, element_size: int, with_scale: bool = False):
        dt = self._dtype(element_size)
        if element_size not in self._ops:
            self._ops[element_size] = All2AllSingle(self.pg, self.max_m, self.n_dim, self.world, dt)
        x = self._inputs[element_size][: int(input_size[0])]
        cs = input_split_cumsum.to(torch.int64)
        splits = torch.diff(cs, prepend=torch.zeros(1, dtype=cs.dtype, device=cs.device))[: self.world]
        osp = torch.empty(self.world, dtype=torch.int32, device=x.device)
        out = self._ops[element_size].forward(x, None, splits, osp)
        return out, osp


class TransportOp:
    """``copy_by_sm``: copy a tensor into rank ``tgt``'s symmetric buffer with a copy kernel
    (reference: ``flux.TransportOp``)."""

    def __init__(self, rank: int, world_size: int, buffer: torch.Tensor, pg=None):
        from ..parallel.symm import SymmBuffer
        self.pg = pg if pg is not None else dist.group.WORLD
        self.rank, self.world = rank, world_size
        self.template = buffer
        self.buf = SymmBuffer(buffer.numel() * buffer.element_size(), self.pg)

    def local_buffer(self) -> torch.Tensor:
        return self.buf.view(self.rank, self.template.dtype, tuple(self.template.shape))

    def copy_by_sm(self, src: torch.Tensor, tgt_rank: int) -> None:
        nbytes = src.numel() * src.element_size()
        if not src.is_cuda:
            self.buf.view(tgt_rank, src.dtype, tuple(src.shape)).copy_(src)
            return
        rc = _native.lib().fluxb_copy_bytes(ctypes.c_void_p(self.buf.ptr(tgt_rank)), ctypes.c_void_p(src.data_ptr()),
                                            ctypes.c_int64(nbytes),
                                            ctypes.c_void_p(_dense.current_stream_ptr(src.device)))
        _native.check(rc, "fluxb_copy_bytes")


def _multi_node(name: str):
    class _Unavailable:
        def __init__(self, *a, **k):
            raise NotImplementedError(
                f"{name}: multi-node operation is outside the single NVSwitch domain this library targets")
        def _no(self, *a, **k):
            raise NotImplementedError(f"{name}: multi-node operation is not built")

        forward = gemm_only = copy_local = reset_signals = _no
    _Unavailable.__name__ = name
    return _Unavailable


GemmRSInterNode = _multi_node("GemmRSInterNode")
GemmRS_multinode = _multi_node("GemmRS_multinode")
AGKernelInterNode = _multi_node("AGKernelInterNode")
AGKernelXNode = _multi_node("AGKernelXNode")


def _taco(name: str):
    class _Unavailable:
        def __init__(self, *a, **k):
            raise NotImplementedError(
                f"{name}: the compressed (TACO) reduce-scatter of the reference fork is a research add-on "
                "for sm80 links and is not built; GemmRS moves bf16 partial tiles over NVLink")
    _Unavailable.__name__ = name
    return _Unavailable


GemmRSTaco = _taco("GemmRSTaco")
GemmRSTacoDoubleBuffered = _taco("GemmRSTacoDoubleBuffered")


def load_tuning_record(record) -> None:
    """Add a tuning record (``TuningRecord`` or dict with ``key`` = [M, N, K] and ``best``) to the
    in-memory table (reference: ``flux.load_tuning_record``)."""
    from ..tuning import table
    key = tuple(record["key"] if isinstance(record, dict) else record.key.get("mnk", ()))
    best = record["best"] if isinstance(record, dict) else record.best
    if len(key) != 3:
        raise ValueError("tuning record needs key = [M, N, K]")
    table.DENSE_TABLE[key] = dict(best)


def bsr_reduce(input: torch.Tensor, output: torch.Tensor, block_h: int = 128, block_w: int = 128) -> torch.Tensor:
    """output[M, N] = sum over dim 0 of input[B, M, N] (reference: ``flux.bsr_reduce``; the block
    sizes only shaped the reference kernel's grid)."""
    if (input.is_cuda and input.dtype in (torch.bfloat16, torch.float16) and input.dtype == output.dtype
            and input.is_contiguous() and output.is_contiguous() and input.shape[-1] % 8 == 0):
        B, M, N = input.shape
        rc = _native.lib().fluxb_rows_sum(ctypes.c_void_p(input.data_ptr()), None, ctypes.c_void_p(output.data_ptr()),
                                          ctypes.c_int64(M), ctypes.c_int(N), ctypes.c_int(B), ctypes.c_int64(M),
                                          ctypes.c_int(_dense.dtype_code(input.dtype)),
                                          ctypes.c_void_p(_dense.current_stream_ptr(input.device)))
        _native.check(rc, "fluxb_rows_sum")
        return output
    output.copy_(input.float().sum(0).to(output.dtype))
    return output


def pad_m_to_TPxTile(input: torch.Tensor, tp_size: int, tile: int = 128) -> torch.Tensor:
    """Pad the rows of ``input`` to a multiple of tp_size * tile (reference: ``pad_m_to_TPxTile``;
    the kernels here clip partial tiles themselves, so callers rarely need it)."""
    m = input.shape[0]
    unit = tp_size * tile
    pm = (-m) % unit
    return torch.nn.functional.pad(input, (0, 0, 0, pm)) if pm else input
