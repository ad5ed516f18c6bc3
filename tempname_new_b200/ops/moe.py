"""MoE layers with the collectives fused in.

* ``GemmGroupedV3AGScatter`` (layer 0): ``out[rows_ep, ffn/TP] = index_select(all_gather(x),
  gather_index) @ W_e^T`` per local expert. One kernel pushes the token shards to all peers,
  gathers rows by routing index inside the A loader and walks a device-built schedule ordered by
  source rank (own shard first), so no routing data visits the host. Reference:
  ``flux.GemmGroupedV3AGScatter`` (``src/pybind/gemm_grouped_v3_ag_scatter.cc:29-68``,
  ``src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc``), which synchronises with the host
  to build its problem list.
* ``GemmGroupedV3GatherRS`` (layer 1): per-expert GEMM with the gate weight applied in the
  epilogue. With whole experts per rank (no tensor parallelism inside an expert) the epilogue
  stores every row straight into the slot ``[token][k]`` of the token owner's staging buffer over
  NVLink and the tail of the same kernel adds each token's top-k slots: one launch, the
  expert-sorted product never exists in memory. With experts split over ranks a second kernel
  sums every token's local top-k rows, sends the partial to the token's owner and lets the owner
  add the W partials. Reference:
  ``flux.GemmGroupedV3GatherRS`` (``src/pybind/gemm_grouped_v3_gather_rs.cc:35-126``,
  ``src/moe_gather_rs``), ``TopkReduceScatterOp``.

Routing tensors follow ``python/flux/testing/moe_utils.py`` of the reference: ``splits =
bincount(experts)``, ``scatter_index[t, k]`` = row of entry (t, k) in the stable expert-sorted
order. ``moe_layer0_torch`` / ``moe_layer1_torch`` state the two layers in PyTorch (CPU path and
test oracle).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Union

import torch
import torch.distributed as dist

from .. import _native
from . import _dense
from ._fused_base import OFF_CTR, OFF_LOCAL, OFF_START, FusedOpBase
from ..parallel.dist_env import DistEnvTPWithEP, MoeArguments
from ..parallel.symm import SymmBuffer, _ELEM

_VP = ctypes.c_void_p
_R = _dense.MAX_RANKS


class MoeGemmArgs(ctypes.Structure):
    _fields_ = [
        ("splits", _VP), ("scatter_index", _VP), ("gather_index", _VP), ("n_entries", ctypes.c_int64),
        ("E", ctypes.c_int32), ("e0", ctypes.c_int32), ("E_local", ctypes.c_int32), ("topk", ctypes.c_int32),
        ("tokens_per_rank", ctypes.c_int32), ("gathered", ctypes.c_int32), ("do_allgather", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32),
        ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("a", _VP), ("a_rows", ctypes.c_int64), ("a_tokens", _VP), ("a_sorted", _VP),
        ("a_sorted_rows", ctypes.c_int64), ("weights", _VP),
        ("d", _VP), ("ldd", ctypes.c_int64),
        ("expert_scale", _VP), ("scalar_scale", _VP), ("row_scale", _VP), ("scratch", _VP),
        ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64), ("status", _VP),
        ("ag_src", _VP), ("ag_land", _VP * _R), ("ag_flags", _VP * _R), ("start_ctr", _VP * _R),
        ("local_cnt", _VP), ("stream", _VP),
        ("scatter", ctypes.c_int32), ("reserved2", ctypes.c_int32),
        ("routing_idx", _VP), ("row_entry", _VP),
        ("sc_stage", _VP * _R), ("sc_flags", _VP * _R), ("sc_out", _VP),
    ]


class MoeCombineArgs(ctypes.Structure):
    _fields_ = [
        ("y", _VP), ("hdr", _VP), ("routing_idx", _VP),
        ("topk", ctypes.c_int32), ("tokens_per_rank", ctypes.c_int32), ("H", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64), ("status", _VP),
        ("stage", _VP * _R), ("flags", _VP * _R), ("start_ctr", _VP * _R),
        ("local_cnt", _VP), ("out", _VP), ("stream", _VP),
    ]


def _out16(dt: torch.dtype) -> torch.dtype:
    """Output dtype of the grouped kernel: the 16-bit input dtype, bf16 for 8-bit inputs."""
    return dt if dt in (torch.bfloat16, torch.float16) else torch.bfloat16


def _f32(t: Optional[torch.Tensor], dev) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.to(device=dev, dtype=torch.float32).contiguous()


def _scratch(E: int, world: int, dev) -> torch.Tensor:
    lib = _native.lib()
    lib.fluxb_moe_schedule_scratch_bytes.restype = ctypes.c_int64
    return torch.zeros(int(lib.fluxb_moe_schedule_scratch_bytes(E, world)), dtype=torch.uint8, device=dev)


def _hdr_ptr(scratch: torch.Tensor, E: int, world: int) -> int:
    lib = _native.lib()
    lib.fluxb_moe_hdr_offset.restype = ctypes.c_int64
    return scratch.data_ptr() + int(lib.fluxb_moe_hdr_offset(E, world))


# ------------------------------------------------------------------------------------------
# PyTorch statements
# ------------------------------------------------------------------------------------------
def moe_layer0_torch(tokens: torch.Tensor, weights: torch.Tensor, splits: torch.Tensor,
                     scatter_index: torch.Tensor, e0: int, output_scale: Optional[torch.Tensor] = None,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """tokens [T, H] (already gathered), weights [E_local, N, H] -> [rows of experts e0.., N]."""
    topk = scatter_index.shape[1]
    n = scatter_index.numel()
    gather = torch.empty(n, dtype=torch.long, device=tokens.device)
    gather[scatter_index.reshape(-1).long()] = torch.arange(n, device=tokens.device) // topk
    offs = torch.cat([torch.zeros(1, dtype=torch.long, device=splits.device), splits.long().cumsum(0)]).tolist()
    outs = []
    for el in range(weights.shape[0]):
        rows = gather[offs[e0 + el]:offs[e0 + el + 1]]
        y = tokens[rows].float() @ weights[el].float().t()
        if output_scale is not None:
            y = y * output_scale[el].float()
        outs.append(y)
    return torch.cat(outs).to(out_dtype or tokens.dtype)


def moe_layer1_partial_torch(x: torch.Tensor, weights: torch.Tensor, splits: torch.Tensor, routing_idx: torch.Tensor,
                             topk: int, e0: int, input_scale=None, weight_scale=None, output_vec_scale=None
                             ) -> torch.Tensor:
    """This rank's contribution to every token: [tokens, H] fp32 (before the reduce-scatter)."""
    offs = torch.cat([torch.zeros(1, dtype=torch.long, device=splits.device), splits.long().cumsum(0)]).tolist()
    base = offs[e0]
    ys = []
    for el in range(weights.shape[0]):
        lo, hi = offs[e0 + el] - base, offs[e0 + el + 1] - base
        y = x[lo:hi].float() @ weights[el].float().t()
        if weight_scale is not None:
            y = y * weight_scale[el].float()
        ys.append(y)
    y = torch.cat(ys)
    if input_scale is not None:
        y = y * input_scale.float().reshape(-1)[0]
    if output_vec_scale is not None:
        y = y * output_vec_scale.float()[:, None]
    y = y.to(x.dtype).float()                       # the kernel stores 16-bit rows before combining
    tokens = routing_idx.numel() // topk
    full = torch.zeros(tokens, weights.shape[1], dtype=torch.float32, device=x.device)
    r = routing_idx.reshape(tokens, topk).long() - base
    ok = (r >= 0) & (r < y.shape[0])
    for k in range(topk):
        sel = ok[:, k]
        full[sel] += y[r[sel, k]]
    return full


# ------------------------------------------------------------------------------------------
class GemmGroupedV3AGScatter(FusedOpBase):
    def __init__(self, tp_env: DistEnvTPWithEP, moe_args: MoeArguments, timeout_s: Optional[float] = None):
        super().__init__(tp_env.tp_group, tp_env.nnodes, timeout_s)
        self.env, self.args = tp_env, moe_args
        if moe_args.nexperts % tp_env.ep_size:
            raise ValueError("experts must divide over the expert-parallel groups")
        self.E = moe_args.nexperts
        self.E_local = self.E // tp_env.ep_size
        self.e0 = tp_env.ep_rank * self.E_local
        self.topk = moe_args.topk
        self.max_tokens = moe_args.max_ntokens
        self.land = SymmBuffer(self.max_tokens * moe_args.hidden * _ELEM[moe_args.input_dtype], self.pg) \
            if self.world > 1 else None
        self._scratch = None
        self._gather = None
        self._sorted = None
        self._sorted_complete = False

    def clear_buffers(self) -> None:
        """Kept for API compatibility: flags carry the call number, nothing needs clearing."""

    def forward(self, inputs_shard, weights, splits_gpu, scatter_index, output_scale=None, outputs_buf=None,
                allgather_output=None, fast_accum: bool = False, sm_margin: int = 0):
        outs = self.forward_multiple_weights(
            inputs_shard, [weights], splits_gpu, scatter_index,
            None if output_scale is None else [output_scale],
            None if outputs_buf is None else [outputs_buf], allgather_output, fast_accum, sm_margin)
        return outs[0]

    def forward_multiple_weights(self, inputs_shard, weights: Sequence[torch.Tensor], splits_gpu, scatter_index,
                                 output_scale: Optional[Sequence[torch.Tensor]] = None,
                                 outputs_buf: Optional[Sequence[torch.Tensor]] = None, allgather_output=None,
                                 fast_accum: bool = False, sm_margin: int = 0) -> List[torch.Tensor]:
        tpr, H = inputs_shard.shape
        tokens = tpr * self.world
        if tokens > self.max_tokens:
            raise ValueError(f"op was built for {self.max_tokens} tokens, got {tokens}")
        topk = scatter_index.shape[-1] if scatter_index.dim() == 2 else self.topk
        if not inputs_shard.is_cuda:
            return self._forward_cpu(inputs_shard, weights, splits_gpu, scatter_index.reshape(tokens, topk),
                                     output_scale, outputs_buf, allgather_output)
        dev = inputs_shard.device
        x = inputs_shard if inputs_shard.is_contiguous() else inputs_shard.contiguous()
        splits = splits_gpu.to(device=dev, dtype=torch.int32).contiguous()
        sidx = scatter_index.reshape(-1).to(torch.int32).contiguous()
        if self._scratch is None:
            self._scratch = _scratch(self.E, self.world, dev)
        if self._gather is None or self._gather.numel() < sidx.numel():
            self._gather = torch.empty(sidx.numel(), dtype=torch.int32, device=dev)
        if outputs_buf is None:
            # sizing the result needs this rank's row count on the host: one small D2H sync that
            # callers avoid by passing outputs_buf
            rows_ep = int(splits[self.e0:self.e0 + self.E_local].sum().item())
        outs = []
        keep = []
        for g, w in enumerate(weights):
            if w.dim() != 3 or w.shape[0] != self.E_local or w.shape[2] != H or not w.is_contiguous():
                raise ValueError("weights must be contiguous [E_local, N, hidden]")
            N = w.shape[1]
            out = outputs_buf[g] if outputs_buf is not None else torch.empty(
                (rows_ep, N), dtype=self.args.output_dtype, device=dev)
            a = MoeGemmArgs()
            a.splits, a.scatter_index, a.gather_index = splits.data_ptr(), sidx.data_ptr(), self._gather.data_ptr()
            a.n_entries = sidx.numel()
            a.E, a.e0, a.E_local, a.topk = self.E, self.e0, self.E_local, topk
            a.tokens_per_rank, a.gathered = tpr, 1
            a.in_dtype = _dense.dtype_code(x.dtype)
            a.N, a.K = N, H
            a.weights, a.d, a.ldd = w.data_ptr(), out.data_ptr(), out.stride(0)
            # Weight groups after the first (gate | up | ...) multiply the same rows: the first
            # launch left them, gathered and expert-sorted, in the sorted buffer, so the others
            # are plain grouped GEMMs on that buffer - no second all-gather, index build or gather
            # (reference: forward_multiple_weights runs one gathered A against all groups,
            # src/moe_ag_scatter/ths_op/gemm_grouped_v3_ag_scatter.cc:461-470)
            reuse_sorted = g > 0 and self._sorted_complete
            sc = _f32(output_scale[g], dev) if output_scale is not None and output_scale[g] is not None else None
            keep.append(sc)
            a.expert_scale = sc.data_ptr() if sc is not None else None
            a.scratch = self._scratch.data_ptr()
            a.rank, a.world = self.rank, self.world
            a.timeout_ns, a.status = int(self.timeout_s * 1e9), self.status.data_ptr()
            a.stream = _dense.current_stream_ptr(dev)
            # expert-sorted copy of this rank's rows, filled by the kernel's communication warps
            rows_cap = out.shape[0]
            if self._sorted is None or self._sorted.shape[0] < rows_cap or self._sorted.shape[1] != H:
                self._sorted = torch.empty((max(rows_cap, 128), H), dtype=x.dtype, device=dev)
            a.a_sorted, a.a_sorted_rows = self._sorted.data_ptr(), self._sorted.shape[0]
            a.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
            if reuse_sorted:
                a.gathered = 0
                a.a, a.a_rows = self._sorted.data_ptr(), self._sorted.shape[0]
                a.scatter_index = a.gather_index = a.a_sorted = None
                _native.check(_native.lib().fluxb_moe_grouped_gemm(ctypes.byref(a)), "fluxb_moe_grouped_gemm")
                outs.append(out)
                continue
            self._begin_call()
            a.epoch = self.epoch
            if self.world > 1:
                a.a_tokens = self.land.ptr(self.rank)
                if g == 0:
                    a.do_allgather = 1
                    a.ag_src = x.data_ptr()
                    for r in range(self.world):
                        a.ag_land[r] = self.land.ptr(r)
                        a.ag_flags[r] = self.ctrl.ptr(r, OFF_CTR)
                        a.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
            else:
                a.a_tokens = x.data_ptr()
            _native.check(_native.lib().fluxb_moe_grouped_gemm(ctypes.byref(a)), "fluxb_moe_grouped_gemm")
            # (the in-loader gather variants selected by FLUXB_MOE_GATHER do not fill the sorted buffer)
            self._sorted_complete = os.environ.get("FLUXB_MOE_GATHER", "") in ("", "pregather")
            outs.append(out)
        if allgather_output is not None:
            if self.world > 1:
                allgather_output.copy_(self.land.view(self.rank, x.dtype, (tokens, H)))
            else:
                allgather_output.copy_(x)
        self._after_launch()
        return outs

    def _forward_cpu(self, x, weights, splits, scatter_index, output_scale, outputs_buf, allgather_output):
        parts = [torch.empty_like(x) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(parts, x.contiguous(), group=self.pg)
        else:
            parts = [x]
        tokens = torch.cat(parts)
        if allgather_output is not None:
            allgather_output.copy_(tokens)
        outs = []
        for g, w in enumerate(weights):
            sc = output_scale[g] if output_scale is not None else None
            y = moe_layer0_torch(tokens, w, splits, scatter_index, self.e0, sc, self.args.output_dtype)
            if outputs_buf is not None:
                outputs_buf[g].copy_(y)
                y = outputs_buf[g]
            outs.append(y)
        return outs

    def profiling(self, inputs_shard, weights, splits_gpu, scatter_index, output_scale=None, outputs_buf=None,
                  allgather_output=None, fast_accum=False, sm_margin=0, prof_ctx=None):
        from ..tuning.profiling import profile_call
        return profile_call(self, "moe_ag_scatter", lambda: self.forward(
            inputs_shard, weights, splits_gpu, scatter_index, output_scale, outputs_buf), prof_ctx)


class GemmGroupedV3GatherRS(FusedOpBase):
    def __init__(self, total_num_experts: int, max_m: int, n_dim: int, topk: int, rank: int, world_size: int,
                 tp_world_size: int, ep_world_size: int, max_input_groups: int = 1, ep_in_dp: bool = False,
                 tp_group=None, dtype: torch.dtype = torch.bfloat16, timeout_s: Optional[float] = None):
        super().__init__(tp_group, 1, timeout_s)
        if world_size != self.world or rank != self.rank:
            raise ValueError("rank / world_size must describe the process group the op runs on")
        if tp_world_size * ep_world_size != world_size or total_num_experts % ep_world_size:
            raise ValueError("tp_world_size * ep_world_size must equal world_size and divide the experts")
        self.E, self.topk, self.H = total_num_experts, topk, n_dim
        self.E_local = self.E // ep_world_size
        self.e0 = (rank // tp_world_size) * self.E_local
        self.max_m = max_m                           # rows of the full problem: tokens * topk
        self.max_tpr = max_m // topk // world_size
        self.dtype = dtype
        # whole experts per rank: the fused path, staging [tokens / W][topk][H] per rank; experts split
        # over ranks: partial sums per source, [W][tokens / W][H]
        self.fused = tp_world_size == 1
        slots = max(world_size, topk) if self.fused else world_size
        self.stage = SymmBuffer(slots * self.max_tpr * n_dim * _ELEM[dtype], self.pg) \
            if (self.world > 1 or self.fused) else None
        self._scratch = None
        self._row_entry = None

    def ep_zero_buffer(self) -> None:
        """Kept for API compatibility: nothing needs zeroing between calls."""

    def forward_gather_rs(self, input, weight, splits_cpu, routing_idx, n_tokens_per_rank=None, input_scale=None,
                          weight_scale=None, output_vec_scale=None, fast_accum: bool = False, sm_margin: int = 0,
                          with_stream_sync: bool = False) -> torch.Tensor:
        return self.forward_gather_rs_multiple([input], [weight], splits_cpu, routing_idx, n_tokens_per_rank,
                                               None if input_scale is None else [input_scale],
                                               None if weight_scale is None else [weight_scale],
                                               None if output_vec_scale is None else [output_vec_scale],
                                               fast_accum, sm_margin, with_stream_sync)

    forward_gather_rs_no_zerobuffer = forward_gather_rs

    def forward_gather_rs_multiple(self, input: Sequence[torch.Tensor], weight: Sequence[torch.Tensor], splits_cpu,
                                   routing_idx, n_tokens_per_rank=None, input_scale=None, weight_scale=None,
                                   output_vec_scale=None, fast_accum: bool = True, sm_margin: int = 0,
                                   with_stream_sync: bool = False) -> torch.Tensor:
        """inputs[g] [rows_ep, ffn_g], weights[g] [E_local, H, ffn_g], routing_idx [tokens*topk] ->
        [tokens / W, H]: sum over groups, top-k entries and ranks."""
        x0 = input[0]
        ridx = routing_idx.reshape(-1)
        tokens = ridx.numel() // self.topk
        tpr = tokens // self.world
        if tpr > self.max_tpr:
            raise ValueError("more tokens than the op was built for")
        if not x0.is_cuda:
            return self._forward_cpu(input, weight, splits_cpu, ridx, tpr, input_scale, weight_scale, output_vec_scale)
        dev = x0.device
        splits = splits_cpu.to(device=dev, dtype=torch.int32, non_blocking=True).contiguous()
        ridx = ridx.to(device=dev, dtype=torch.int32).contiguous()
        if self._scratch is None:
            self._scratch = _scratch(self.E, self.world, dev)
        rows_ep = x0.shape[0]
        if self.fused and len(input) == 1 and rows_ep > 0:
            return self._forward_fused(x0, weight[0], splits, ridx, tpr,
                                       input_scale[0] if input_scale is not None else None,
                                       weight_scale[0] if weight_scale is not None else None,
                                       output_vec_scale[0] if output_vec_scale is not None else None)
        y = None
        keep = []
        for g, (x, w) in enumerate(zip(input, weight)):
            if w.dim() != 3 or w.shape[0] != self.E_local or w.shape[1] != self.H or not w.is_contiguous():
                raise ValueError("weights must be contiguous [E_local, n_dim, ffn]")
            x = x if x.is_contiguous() else x.contiguous()
            yg = torch.empty((max(rows_ep, 1), self.H), dtype=_out16(x.dtype), device=dev)
            a = MoeGemmArgs()
            a.splits = splits.data_ptr()
            a.E, a.e0, a.E_local, a.topk = self.E, self.e0, self.E_local, self.topk
            a.tokens_per_rank, a.gathered = tpr, 0
            a.in_dtype = _dense.dtype_code(x.dtype)
            a.N, a.K = self.H, x.shape[1]
            a.a, a.a_rows = x.data_ptr(), max(rows_ep, 1)
            a.weights, a.d, a.ldd = w.data_ptr(), yg.data_ptr(), self.H
            ws = _f32(weight_scale[g], dev) if weight_scale is not None and weight_scale[g] is not None else None
            isc = _f32(input_scale[g], dev) if input_scale is not None and input_scale[g] is not None else None
            ovs = _f32(output_vec_scale[g], dev) if output_vec_scale is not None and output_vec_scale[g] is not None else None
            keep += [ws, isc, ovs]
            a.expert_scale = ws.data_ptr() if ws is not None else None
            a.scalar_scale = isc.data_ptr() if isc is not None else None
            a.row_scale = ovs.data_ptr() if ovs is not None else None
            a.scratch = self._scratch.data_ptr()
            a.rank, a.world = self.rank, self.world
            a.timeout_ns, a.status = int(self.timeout_s * 1e9), self.status.data_ptr()
            a.stream = _dense.current_stream_ptr(dev)
            _native.check(_native.lib().fluxb_moe_grouped_gemm(ctypes.byref(a)), "fluxb_moe_grouped_gemm")
            y = yg if y is None else y.add_(yg)
        out = torch.empty((tpr, self.H), dtype=y.dtype, device=dev)
        self._combine(y, ridx, tpr, out)
        self._after_launch()
        return out

    def _forward_fused(self, x, w, splits, ridx, tpr, input_scale, weight_scale, output_vec_scale) -> torch.Tensor:
        """One launch: grouped GEMM whose epilogue scatters the gate-weighted rows to the token
        owners' [token][k] slots and whose tail adds the top-k slots of the local tokens."""
        dev = x.device
        if w.dim() != 3 or w.shape[0] != self.E_local or w.shape[1] != self.H or not w.is_contiguous():
            raise ValueError("weights must be contiguous [E_local, n_dim, ffn]")
        x = x if x.is_contiguous() else x.contiguous()
        rows_ep = x.shape[0]
        if self._row_entry is None or self._row_entry.numel() < rows_ep:
            self._row_entry = torch.empty(max(rows_ep, self.max_m // max(self.world, 1)), dtype=torch.int32, device=dev)
        out = torch.empty((tpr, self.H), dtype=_out16(x.dtype), device=dev)
        self._begin_call()
        a = MoeGemmArgs()
        a.splits = splits.data_ptr()
        a.E, a.e0, a.E_local, a.topk = self.E, self.e0, self.E_local, self.topk
        a.tokens_per_rank, a.gathered = tpr, 0
        a.in_dtype = _dense.dtype_code(x.dtype)
        a.N, a.K = self.H, x.shape[1]
        a.a, a.a_rows = x.data_ptr(), rows_ep
        a.weights, a.d, a.ldd = w.data_ptr(), None, self.H
        ws = _f32(weight_scale, dev) if weight_scale is not None else None
        isc = _f32(input_scale, dev) if input_scale is not None else None
        ovs = _f32(output_vec_scale, dev) if output_vec_scale is not None else None
        a.expert_scale = ws.data_ptr() if ws is not None else None
        a.scalar_scale = isc.data_ptr() if isc is not None else None
        a.row_scale = ovs.data_ptr() if ovs is not None else None
        a.scratch = self._scratch.data_ptr()
        a.rank, a.world, a.epoch = self.rank, self.world, self.epoch
        a.timeout_ns, a.status = int(self.timeout_s * 1e9), self.status.data_ptr()
        a.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        a.scatter = 1
        a.n_entries = ridx.numel()
        a.routing_idx, a.row_entry = ridx.data_ptr(), self._row_entry.data_ptr()
        for r in range(self.world):
            a.sc_stage[r] = self.stage.ptr(r)
            a.sc_flags[r] = self.ctrl.ptr(r, OFF_CTR)
            a.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
        a.sc_out = out.data_ptr()
        a.stream = _dense.current_stream_ptr(dev)
        _native.check(_native.lib().fluxb_moe_grouped_gemm(ctypes.byref(a)), "fluxb_moe_grouped_gemm")
        self._after_launch()
        return out

    def _combine(self, y: torch.Tensor, ridx: torch.Tensor, tpr: int, out: torch.Tensor) -> None:
        self._begin_call()
        c = MoeCombineArgs()
        c.y, c.routing_idx = y.data_ptr(), ridx.data_ptr()
        c.hdr = _hdr_ptr(self._scratch, self.E, self.world)
        c.topk, c.tokens_per_rank, c.H = self.topk, tpr, self.H
        c.dtype = _dense.dtype_code(y.dtype)
        c.rank, c.world, c.epoch = self.rank, self.world, self.epoch
        c.timeout_ns, c.status = int(self.timeout_s * 1e9), self.status.data_ptr()
        c.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        if self.world > 1:
            for r in range(self.world):
                c.stage[r] = self.stage.ptr(r)
                c.flags[r] = self.ctrl.ptr(r, OFF_CTR)
                c.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
        else:
            if getattr(self, "_solo_stage", None) is None or self._solo_stage.numel() < tpr * self.H:
                self._solo_stage = torch.empty(tpr * self.H, dtype=y.dtype, device=y.device)
            c.stage[0] = self._solo_stage.data_ptr()
            c.flags[0] = self.ctrl.ptr(0, OFF_CTR)
            c.start_ctr[0] = self.ctrl.ptr(0, OFF_START)
        c.out = out.data_ptr()
        c.stream = _dense.current_stream_ptr(y.device)
        _native.check(_native.lib().fluxb_moe_combine(ctypes.byref(c)), "fluxb_moe_combine")

    def _forward_cpu(self, inputs, weights, splits, ridx, tpr, input_scale, weight_scale, output_vec_scale):
        full = None
        for g, (x, w) in enumerate(zip(inputs, weights)):
            part = moe_layer1_partial_torch(
                x, w, splits, ridx, self.topk, self.e0,
                input_scale[g] if input_scale is not None else None,
                weight_scale[g] if weight_scale is not None else None,
                output_vec_scale[g] if output_vec_scale is not None else None)
            full = part if full is None else full + part
        full = full.to(inputs[0].dtype)
        out = torch.empty(tpr, full.shape[1], dtype=full.dtype)
        if self.world > 1:
            dist.reduce_scatter(out, list(full.chunk(self.world)), group=self.pg)
        else:
            out = full
        return out

    def profiling(self, input, weight, splits_cpu, routing_idx, n_tokens_per_rank=None, input_scale=None,
                  weight_scale=None, output_vec_scale=None, fast_accum=False, sm_margin=0, with_stream_sync=False,
                  prof_ctx=None):
        from ..tuning.profiling import profile_call
        return profile_call(self, "moe_gather_rs", lambda: self.forward_gather_rs(
            input, weight, splits_cpu, routing_idx, n_tokens_per_rank, input_scale, weight_scale, output_vec_scale),
            prof_ctx)


class GemmGroupedV3:
    """Per-expert GEMM without communication: ``forward(input [rows, K], splits_cpu [E])`` with
    ``weight [E, N, K]`` (reference: ``flux.GemmGroupedV3``, ``src/pybind/gemm_only.cc:171-197``)."""

    def __init__(self, weight: torch.Tensor, num_experts: int):
        if weight.dim() != 3 or weight.shape[0] != num_experts:
            raise ValueError("weight must be [num_experts, N, K]")
        self.weight = weight.contiguous()
        self.E = num_experts
        self._scratch = None
        self._status = None

    def forward(self, input: torch.Tensor, splits_cpu: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                weight_scale: Optional[torch.Tensor] = None, output_scale: Optional[torch.Tensor] = None,
                fast_accum: bool = False, sm_margin: int = 0) -> torch.Tensor:
        """``input_scale`` [1] and ``weight_scale`` [E] (one per expert) multiply the product, as in the
        reference's ``GemmGroupedV2.forward`` (src/pybind/gemm_only.cc:171-190); ``output_scale`` is
        accepted and, as there for 16-bit outputs, not applied."""
        N = self.weight.shape[1]
        if not input.is_cuda:
            outs, row = [], 0
            for e, n in enumerate(splits_cpu.tolist()):
                y = input[row:row + n].float() @ self.weight[e].float().t()
                if weight_scale is not None:
                    y = y * weight_scale.reshape(-1)[e].float()
                if input_scale is not None:
                    y = y * input_scale.reshape(-1)[0].float()
                outs.append(y)
                row += n
            return torch.cat(outs).to(input.dtype)
        dev = input.device
        if self._scratch is None:
            self._scratch = _scratch(self.E, 1, dev)
            self._status = torch.zeros(4, dtype=torch.int32, device=dev)
        splits = splits_cpu.to(device=dev, dtype=torch.int32, non_blocking=True).contiguous()
        x = input if input.is_contiguous() else input.contiguous()
        out = torch.empty((x.shape[0], N), dtype=_out16(x.dtype), device=dev)
        a = MoeGemmArgs()
        a.splits = splits.data_ptr()
        a.E, a.e0, a.E_local, a.topk = self.E, 0, self.E, 1
        a.in_dtype = _dense.dtype_code(x.dtype)
        a.N, a.K = N, x.shape[1]
        a.a, a.a_rows = x.data_ptr(), x.shape[0]
        a.weights, a.d, a.ldd = self.weight.data_ptr(), out.data_ptr(), N
        ws = _f32(weight_scale, dev) if weight_scale is not None else None
        isc = _f32(input_scale, dev) if input_scale is not None else None
        a.expert_scale = ws.data_ptr() if ws is not None else None
        a.scalar_scale = isc.data_ptr() if isc is not None else None
        a.scratch = self._scratch.data_ptr()
        a.rank, a.world = 0, 1
        a.status = self._status.data_ptr()
        a.stream = _dense.current_stream_ptr(dev)
        _native.check(_native.lib().fluxb_moe_grouped_gemm(ctypes.byref(a)), "fluxb_moe_grouped_gemm")
        return out

    __call__ = forward

    def profiling(self, input: torch.Tensor, splits_cpu: torch.Tensor, prof_ctx=None) -> torch.Tensor:
        from ..tuning.profiling import profile_call
        return profile_call(self, "gemm_grouped_v3", lambda: self.forward(input, splits_cpu), prof_ctx)


class GemmGroupedV2(GemmGroupedV3):
    """Same kernel behind the reference's older constructor:
    ``GemmGroupedV2(weight, num_experts, in_type, out_type)``."""

    def __init__(self, weight: torch.Tensor, num_experts: int, in_type: Optional[torch.dtype] = None,
                 out_type: Optional[torch.dtype] = None):
        super().__init__(weight, num_experts)
        if in_type is not None and in_type != weight.dtype:
            raise TypeError("in_type must be the dtype of the weights")
        if out_type is not None and out_type != weight.dtype:
            raise NotImplementedError("the grouped kernel writes the input dtype")


GemmGroupedV2AGScatterOp = GemmGroupedV3AGScatter
GemmGroupedV2GatherRSOp = GemmGroupedV3GatherRS
# the reference's Triton entry points of the two MoE ops compute the same results through its Triton
# kernels; here there is one implementation, so the names lead to it
GemmGroupedV3AGScatter.forward_triton_aot = GemmGroupedV3AGScatter.forward
GemmGroupedV3GatherRS.forward_gather_rs_triton_aot = GemmGroupedV3GatherRS.forward_gather_rs


def topk_scatter_reduce(inputs: torch.Tensor, scatter_idx: torch.Tensor, topk: int) -> torch.Tensor:
    """out[t] = sum_k inputs[scatter_idx[t * topk + k]] in fp32 (reference: ``flux.topk_scatter_reduce``,
    src/pybind/gemm_grouped_v3_gather_rs.cc:33). ``inputs`` may be a list of tensors (one per weight
    group), which are added first."""
    if isinstance(inputs, (list, tuple)):
        x = inputs[0] if len(inputs) == 1 else torch.stack([t.float() for t in inputs]).sum(0).to(inputs[0].dtype)
    else:
        x = inputs
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[1] % 8 == 0:
        x = x if x.is_contiguous() else x.contiguous()
        idx = scatter_idx.reshape(-1).to(device=x.device, dtype=torch.int32).contiguous()
        rows = idx.numel() // topk
        out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        rc = _native.lib().fluxb_rows_sum(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(idx.data_ptr()),
                                          ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(rows),
                                          ctypes.c_int(x.shape[1]), ctypes.c_int(topk), ctypes.c_int64(0),
                                          ctypes.c_int(_dense.dtype_code(x.dtype)),
                                          ctypes.c_void_p(_dense.current_stream_ptr(x.device)))
        _native.check(rc, "fluxb_rows_sum")
        return out
    idx = scatter_idx.reshape(-1, topk).long()
    return x[idx].float().sum(1).to(x.dtype)


_PAD_ROW = 2 ** 31 - 1    # marks padding rows of a blocked index (INT32_MAX, as in the reference)


def calc_moe_triton_blocked_gather_a(splits: torch.Tensor, ep_start: int, ep_nexperts: int, block_size_m: int,
                                     gather_a_index: torch.Tensor, expert_index: torch.Tensor, stream=None) -> None:
    """Blocked row index of a grouped GEMM whose row tiles never straddle two experts: the rows of
    every expert in [ep_start, ep_start + ep_nexperts) are padded to a multiple of ``block_size_m``;
    ``gather_a_index[padded row]`` = row inside this rank's expert-sorted rows (INT32_MAX on padding),
    ``expert_index[tile]`` = local expert of the tile. The outputs are written in place, as by the
    reference's kernel of the same name (src/moe_gather_rs/moe_utils.cu:762-793)."""
    sp = splits[ep_start:ep_start + ep_nexperts].to(torch.int64)
    dev = sp.device
    tiles = (sp + block_size_m - 1) // block_size_m
    n_tiles = int(tiles.sum())
    m_start = torch.cumsum(sp, 0) - sp
    tile_start = torch.cumsum(tiles, 0) - tiles
    tile_expert = torch.repeat_interleave(torch.arange(ep_nexperts, device=dev), tiles)
    expert_index[:n_tiles] = tile_expert.to(expert_index.dtype)
    pos = torch.arange(n_tiles * block_size_m, device=dev)
    e = tile_expert[pos // block_size_m]
    i = pos - tile_start[e] * block_size_m                    # row inside the expert, padding included
    rows = torch.where(i < sp[e], m_start[e] + i, torch.full_like(i, _PAD_ROW))
    gather_a_index[:pos.numel()] = rows.to(gather_a_index.dtype)


def prepare_moe_ag_scatter_args(splits_gpu: torch.Tensor, scatter_index: torch.Tensor, ntokens: int, topk: int,
                                num_weight_groups: int, ep_start: int, ep_experts: int, rank: int,
                                world_size: int, tile_size_m: int, cp_stream=None):
    """Index tensors for a tile-blocked MoE layer-0 GEMM over this rank's experts (the arguments the
    reference prepares for its Triton kernel, src/pybind/gemm_grouped_v2_ag_scatter.cc:30). Returns
    ``(M_this_ep, M_this_ep_pad, gather_A_index, scatter_D_index, expert_index, rank_start_index,
    rank_end_index)``: per padded row the token to read (INT32_MAX on padding) and the output row to
    write; per row tile its local expert and the first / last source rank whose tokens it reads, so
    that a consumer can wait for exactly those shards of the all-gather. The kernels of this library
    build the equivalent schedule on the device (``moe_schedule_kernel``); this is the same
    information as tensors."""
    dev = splits_gpu.device
    sp_all = splits_gpu.to(torch.int64)
    base = int(sp_all[:ep_start].sum())
    sp = sp_all[ep_start:ep_start + ep_experts]
    M = int(sp.sum())
    tiles = (sp + tile_size_m - 1) // tile_size_m
    n_tiles = int(tiles.sum())
    M_pad = n_tiles * tile_size_m
    gather_rows = torch.empty(M_pad, dtype=torch.int32, device=dev)
    expert_index = torch.empty(n_tiles, dtype=torch.int32, device=dev)
    calc_moe_triton_blocked_gather_a(splits_gpu, ep_start, ep_experts, tile_size_m, gather_rows, expert_index)
    # sorted row -> token: scatter_index[token, k] is the sorted row of (token, k)
    flat = scatter_index.reshape(-1).to(torch.int64)
    token_of_row = torch.empty(flat.numel(), dtype=torch.int64, device=dev)
    token_of_row[flat] = torch.arange(flat.numel(), device=dev) // topk
    pad = gather_rows == _PAD_ROW
    rows = gather_rows.to(torch.int64).clamp(max=max(M - 1, 0))
    tok = token_of_row[base + rows]
    gather_a = torch.where(pad, torch.full_like(tok, _PAD_ROW), tok).to(torch.int32)
    scatter_d = torch.where(pad, torch.full_like(rows, _PAD_ROW), rows).to(torch.int32)
    tpr = max(ntokens // world_size, 1)
    src = (tok // tpr).reshape(n_tiles, tile_size_m)
    padm = pad.reshape(n_tiles, tile_size_m)
    rank_start = torch.where(padm, torch.full_like(src, world_size), src).min(1).values.to(torch.int32)
    rank_end = torch.where(padm, torch.full_like(src, -1), src).max(1).values.to(torch.int32)
    m_pad_t = torch.tensor([M_pad], dtype=torch.int32, device=dev)
    rep = lambda t: t.repeat(num_weight_groups) if num_weight_groups > 1 else t  # noqa: E731
    return M, m_pad_t, rep(gather_a), rep(scatter_d), rep(expert_index), rep(rank_start), rep(rank_end)
