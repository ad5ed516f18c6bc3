"""Ulysses sequence-parallel attention projections with the all-to-all fused into the GEMM.

* ``GemmAllToAllTranspose`` (pre-attention): QKV projection on the local sequence shard; the GEMM
  epilogue stores every (32 positions x 64 columns) piece directly into the rank that owns the
  head, already in the head-sharded layout. Reference: ``flux.GemmAllToAllTranspose``
  (``src/pybind/gemm_a2a_transpose.cc:30-140``, ``src/gemm_a2a_transpose/``), which writes a local
  GEMM output, flags tiles and runs a separate pull kernel on carved-out SMs.
  The stand-alone exchanges (``pre_attn_a2a``, ``pre_attn_qkv_pack_a2a``, ``post_attn_a2a``) and
  the forms with per-rank sequence lengths run on one strided-exchange kernel over peer memory
  (``fluxb_strided_exchange``, csrc/ops/a2a.cu) instead of a library collective; with per-rank
  lengths the projection and the exchange are two launches.
* ``AllToAllTransposeGemm`` (post-attention): the head-sharded attention output is pushed into
  the peers' GEMM-input buffers by two warps of every CTA while the out-projection GEMM of the
  same kernel walks its K loop one source slice at a time, own slice first. Reference:
  ``flux.AllToAllTransposeGemm`` (``src/pybind/a2a_transpose_gemm.cc:30-137``,
  ``src/a2a_transpose_gemm/``): push kernel + flag-gated consumer GEMM.

Layouts follow ``python/flux/testing/ulysses_sp_utils.py:21-166`` of the reference;
``pre_attn_a2a_torch`` / ``post_attn_a2a_torch`` below restate them with ``all_to_all_single``
and are the CPU path and the test oracle.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native
from . import _dense
from ._fused_base import OFF_CTR, OFF_LOCAL, OFF_START, FusedOpBase
from .gemm_only import _out_dtype, as_nk
from .options import PreAttnAllToAllCommOp
from ..parallel.symm import SymmBuffer, _ELEM

_VP = ctypes.c_void_p


class A2AArgs(ctypes.Structure):
    _fields_ = [
        ("base", _dense.DenseArgs),
        ("bs", ctypes.c_int32), ("local_seq", ctypes.c_int32), ("hd", ctypes.c_int32),
        ("groups", ctypes.c_int32),
        ("group_heads", ctypes.c_int32 * 3),
        ("layout", ctypes.c_int32),
        ("out", (_VP * _dense.MAX_RANKS) * 3),
        ("attn", _VP),
        ("land", _VP * _dense.MAX_RANKS),
        ("a2a_flags", _VP * _dense.MAX_RANKS),
        ("copy_local", ctypes.c_int32),
    ]


class StridedCopy(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("dst", _VP),
        ("n0", ctypes.c_int32), ("n1", ctypes.c_int32), ("n2", ctypes.c_int32), ("vec_bytes", ctypes.c_int32),
        ("ss0", ctypes.c_int64), ("ss1", ctypes.c_int64), ("ss2", ctypes.c_int64),
        ("ds0", ctypes.c_int64), ("ds1", ctypes.c_int64), ("ds2", ctypes.c_int64),
    ]


class ExchangeArgs(ctypes.Structure):
    _fields_ = [
        ("copy", (StridedCopy * 3) * _dense.MAX_RANKS),
        ("ncopies", ctypes.c_int32), ("num_ctas", ctypes.c_int32),
        ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64), ("status", _VP),
        ("flags", _VP * _dense.MAX_RANKS), ("start_ctr", _VP * _dense.MAX_RANKS),
        ("local_cnt", _VP), ("stream", _VP),
    ]


def _strided_exchange(op: FusedOpBase, copies, device, num_ctas: int = 0) -> None:
    """One launch of the strided-exchange kernel on ``op``'s control block. ``copies[d]`` is the list
    (the same length for every d, at most 3) of ``(src_ptr, dst_ptr, (n0, n1, n2), vec_bytes,
    (ss0, ss1, ss2), (ds0, ds1, ds2))`` for destination rank d; strides in bytes."""
    op._begin_call()
    a = ExchangeArgs()
    a.ncopies = len(copies[0])
    a.num_ctas = num_ctas if num_ctas > 0 else 0
    a.rank, a.world, a.epoch = op.rank, op.world, op.epoch
    a.timeout_ns, a.status = int(op.timeout_s * 1e9), op.status.data_ptr()
    for d in range(op.world):
        a.flags[d] = op.ctrl.ptr(d, OFF_CTR)
        a.start_ctr[d] = op.ctrl.ptr(d, OFF_START)
        for g, (src, dst, n, vec, ss, ds) in enumerate(copies[d]):
            c = a.copy[d][g]
            c.src, c.dst = src, dst
            c.n0, c.n1, c.n2 = n
            c.vec_bytes = vec
            c.ss0, c.ss1, c.ss2 = ss
            c.ds0, c.ds1, c.ds2 = ds
    a.local_cnt = op.ctrl.ptr(op.rank, OFF_LOCAL)
    a.stream = _dense.current_stream_ptr(device)
    _native.check(_native.lib().fluxb_strided_exchange(ctypes.byref(a)), "fluxb_strided_exchange")
    op._after_launch()


# ------------------------------------------------------------------------------------------
# PyTorch statements of the two all-to-alls (any backend)
# ------------------------------------------------------------------------------------------
def _a2a_heads(x: torch.Tensor, group, transpose: bool) -> torch.Tensor:
    """x [bs, local_seq, heads, hd] -> [bs, heads/W, seq, hd] (transpose) or [bs, seq, heads/W, hd]."""
    W = dist.get_world_size(group)
    bs, ls, nh, hd = x.shape
    send = x.reshape(bs, ls, W, nh // W, hd).permute(2, 0, 1, 3, 4).contiguous()   # [W, bs, ls, lh, hd]
    recv = torch.empty_like(send)
    if W > 1:
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv = send
    out = recv.permute(1, 0, 2, 3, 4).reshape(bs, W * ls, nh // W, hd)             # [bs, seq, lh, hd]
    return out.permute(0, 2, 1, 3).contiguous() if transpose else out.contiguous()


def pre_attn_a2a_torch(x: torch.Tensor, group, bs: int, local_seq: int, nh: int, hd: int) -> List[torch.Tensor]:
    return [_a2a_heads(x.reshape(bs, local_seq, nh, hd), group, True)]


def pre_attn_qkv_pack_a2a_torch(x: torch.Tensor, group, bs: int, local_seq: int, nh: int, hd: int, gqa: int
                                ) -> List[torch.Tensor]:
    W = dist.get_world_size(group)
    x = x.reshape(bs, local_seq, nh, hd)
    local_nh = nh // W
    lq, lk = local_nh // (gqa + 2) * gqa, local_nh // (gqa + 2)
    q, k, v = x[:, :, :lq * W], x[:, :, lq * W:(lq + lk) * W], x[:, :, (lq + lk) * W:]
    return [_a2a_heads(t.contiguous(), group, False) for t in (q, k, v)]


def post_attn_a2a_torch(x: torch.Tensor, group, a2a_only: bool) -> torch.Tensor:
    """x [bs, heads/W, seq, hd] (or [bs, seq, heads/W, hd] if a2a_only) -> [bs, seq/W, heads*hd]."""
    W = dist.get_world_size(group)
    if not a2a_only:
        x = x.permute(0, 2, 1, 3)
    bs, seq, lh, hd = x.shape
    ls = seq // W
    send = x.reshape(bs, W, ls, lh, hd).permute(1, 0, 2, 3, 4).contiguous()         # [W dst, bs, ls, lh, hd]
    recv = torch.empty_like(send)
    if W > 1:
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv = send
    return recv.permute(1, 2, 0, 3, 4).reshape(bs, ls, W * lh * hd).contiguous()   # heads ordered by source


def _seq_lens_list(seq_lens_cpu, world: int) -> List[int]:
    lens = [int(v) for v in (seq_lens_cpu.tolist() if hasattr(seq_lens_cpu, "tolist") else seq_lens_cpu)]
    if len(lens) != world:
        raise ValueError("seq_lens_cpu needs one length per rank")
    return lens


def pre_attn_a2a_varlen_torch(x: torch.Tensor, group, seq_lens: List[int]) -> torch.Tensor:
    """Ranks hold different sequence lengths (reference: the ``seq_lens_cpu`` / "dp" form of
    python/flux/testing/ulysses_sp_utils.py:46-116). x [bs, seq_lens[rank], heads, hd] ->
    [bs, sum(seq_lens), heads/W, hd], sources in rank order."""
    W, rank = dist.get_world_size(group), dist.get_rank(group)
    bs, ls, nh, hd = x.shape
    lh = nh // W
    send = x.reshape(bs, ls, W, lh, hd).permute(2, 1, 0, 3, 4).contiguous().reshape(W * ls, bs, lh, hd)
    recv = torch.empty((sum(seq_lens), bs, lh, hd), dtype=x.dtype, device=x.device)
    if W > 1:
        dist.all_to_all_single(recv, send, output_split_sizes=list(seq_lens), input_split_sizes=[ls] * W,
                               group=group)
    else:
        recv = send
    assert ls == seq_lens[rank]
    return recv.permute(1, 0, 2, 3).contiguous()


def post_attn_a2a_varlen_torch(x: torch.Tensor, group, a2a_only: bool, seq_lens: List[int]) -> torch.Tensor:
    """x [bs, heads/W, sum(seq_lens), hd] (or [bs, sum, heads/W, hd] if a2a_only) ->
    [bs, seq_lens[rank], heads*hd] (reference: ulysses_sp_utils.py:119-150, ``is_dp``)."""
    W, rank = dist.get_world_size(group), dist.get_rank(group)
    if not a2a_only:
        x = x.permute(0, 2, 1, 3)
    bs, total, lh, hd = x.shape
    ls = seq_lens[rank]
    send = x.permute(1, 0, 2, 3).contiguous()                                      # [sum, bs, lh, hd]
    recv = torch.empty((W * ls, bs, lh, hd), dtype=x.dtype, device=x.device)
    if W > 1:
        dist.all_to_all_single(recv, send, output_split_sizes=[ls] * W, input_split_sizes=list(seq_lens),
                               group=group)
    else:
        recv = send
    return recv.reshape(W, ls, bs, lh, hd).permute(2, 1, 0, 3, 4).reshape(bs, ls, W * lh * hd).contiguous()


_SP_GROUPS = {}


def _sp_group(tp_group, sp_size: int):
    """The sequence-parallel group of this rank: ``tp_group`` itself when ``sp_size`` is its size,
    else the block of ``sp_size`` consecutive ranks of ``tp_group`` that contains this rank
    (reference: ``sp_size`` smaller than the group, src/gemm_a2a_transpose/ths_op/
    gemm_all2all_transpose.cc:145-160). Sub-groups are created once per (group, sp_size); creating
    them is a collective over all processes, so every rank must build its ops in the same order."""
    pg = tp_group if tp_group is not None else dist.group.WORLD
    world = dist.get_world_size(pg)
    if sp_size in (0, None) or sp_size == world:
        return pg
    if sp_size < 1 or world % sp_size:
        raise ValueError("sp_size must divide the size of the process group")
    key = (id(pg), sp_size)
    if key not in _SP_GROUPS:
        ranks = dist.get_process_group_ranks(pg)
        me = dist.get_rank()
        mine = None
        for c in range(world // sp_size):
            block = ranks[c * sp_size:(c + 1) * sp_size]
            sub = dist.new_group(block)
            if me in block:
                mine = sub
        _SP_GROUPS[key] = mine
    return _SP_GROUPS[key]


class GemmAllToAllTranspose(FusedOpBase):
    def __init__(self, tp_group, nnodes: int, sp_size: int, bs: int, seq: int, hidden_dim: int,
                 head_dim: int, n_dim: int, input_dtype: torch.dtype,
                 output_dtype: Optional[torch.dtype] = None, transpose_weight: bool = False, gqa: int = 0,
                 comm_op: PreAttnAllToAllCommOp = PreAttnAllToAllCommOp.A2ATranspose,
                 max_num_comm_buf: int = 1, timeout_s: Optional[float] = None):
        super().__init__(_sp_group(tp_group, sp_size), nnodes, timeout_s)
        self.bs, self.seq, self.hidden, self.hd, self.n_dim = bs, seq, hidden_dim, head_dim, n_dim
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.transpose_weight, self.gqa, self.comm_op = transpose_weight, gqa, PreAttnAllToAllCommOp(comm_op)
        W = self.world
        if seq % W or n_dim % head_dim or (n_dim // head_dim) % W:
            raise ValueError("seq and the head count must divide over the group")
        self.local_seq = seq // W
        self.nh = n_dim // head_dim
        local_nh = self.nh // W
        if self.comm_op == PreAttnAllToAllCommOp.QKVPackA2A:
            lq, lk = local_nh // (gqa + 2) * gqa, local_nh // (gqa + 2)
            if lq + 2 * lk != local_nh or lk == 0:
                raise ValueError("heads per rank must be a multiple of gqa + 2")
            self.group_heads = [lq * W, lk * W, lk * W]
            self.layout = 1     # [bs, seq, heads/W, hd]
        else:
            self.group_heads = [self.nh]
            self.layout = 0     # [bs, heads/W, seq, hd]
        # one symmetric block holds this rank's outputs of every group, back to back
        self.out_elems = [bs * (g // W) * seq * head_dim for g in self.group_heads]
        self.out_buf = SymmBuffer(sum(self.out_elems) * _ELEM[self.output_dtype], self.pg)

    def _out_views(self) -> List[torch.Tensor]:
        W, off, views = self.world, 0, []
        for g, n in zip(self.group_heads, self.out_elems):
            shape = (self.bs, g // W, self.seq, self.hd) if self.layout == 0 else (self.bs, self.seq, g // W, self.hd)
            views.append(self.out_buf.view(self.rank, self.output_dtype, shape, off))
            off += n * _ELEM[self.output_dtype]
        return views

    def forward(self, input: torch.Tensor, weight: torch.Tensor, seq_lens_cpu=None,
                bias: Optional[torch.Tensor] = None, outputs: Optional[List[torch.Tensor]] = None,
                input_scale=None, weight_scale=None, output_scale=None, fast_accum: bool = False,
                num_comm_sm: int = -1, sm_margin: int = 0) -> List[torch.Tensor]:
        """input [bs, seq/W, hidden] -> A2ATranspose: [out [bs, heads/W, seq, hd]];
        QKVPackA2A: [q, k, v], each [bs, seq, heads_x/W, hd]. Without ``outputs`` the results are
        views of the op's symmetric buffer and stay valid until the next call."""
        if seq_lens_cpu is not None:
            return self._forward_varlen(input, weight, _seq_lens_list(seq_lens_cpu, self.world), bias, outputs)
        w = as_nk(weight, self.transpose_weight)
        x2 = input.reshape(self.bs * self.local_seq, self.hidden)
        self._begin_call()
        if not input.is_cuda:
            res = self._forward_cpu(x2, w, bias)
        else:
            x2 = x2 if x2.is_contiguous() else x2.contiguous()
            keep: list = []
            args = A2AArgs()
            base = _dense.base_args(x2, w, bias, self.output_dtype, m=x2.shape[0], status=self.status, keep=keep)
            base.M = x2.shape[0]
            # the all-to-all runs in the epilogue of the GEMM's own CTAs: nothing to carve out for
            # num_comm_sm; sm_margin shrinks the grid
            base.num_sms = self._num_sms(sm_margin)
            base.mode, base.rank, base.world = 3, self.rank, self.world
            base.epoch, base.timeout_ns = self.epoch, int(self.timeout_s * 1e9)
            base.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
            for r in range(self.world):
                base.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
                args.a2a_flags[r] = self.ctrl.ptr(r, OFF_CTR)
            args.base = base
            args.bs, args.local_seq, args.hd = self.bs, self.local_seq, self.hd
            args.groups, args.layout = len(self.group_heads), self.layout
            off = 0
            for g, (heads, n) in enumerate(zip(self.group_heads, self.out_elems)):
                args.group_heads[g] = heads
                for r in range(self.world):
                    args.out[g][r] = self.out_buf.ptr(r, off)
                off += n * _ELEM[self.output_dtype]
            _native.check(_native.lib().fluxb_ulysses_gemm(ctypes.byref(args)), "fluxb_ulysses_gemm")
            self._after_launch()
            res = self._out_views()
        if outputs is not None:
            for dst, src in zip(outputs, res):
                dst.copy_(src)
            return outputs
        return res

    __call__ = forward

    def _forward_varlen(self, input, weight, seq_lens, bias, outputs):
        """Ranks with different sequence lengths: the projection runs on the GEMM kernel, the
        exchange as one variable-split collective of the process group (not fused)."""
        if self.comm_op != PreAttnAllToAllCommOp.QKVPackA2A:
            raise NotImplementedError("per-rank sequence lengths exist for QKVPackA2A only, as in the reference "
                                      "(python/flux/testing/ulysses_sp_utils.py:24-25)")
        w = as_nk(weight, self.transpose_weight)
        ls = seq_lens[self.rank]
        x2 = input.reshape(self.bs * ls, self.hidden)
        if x2.is_cuda:
            x2 = x2 if x2.is_contiguous() else x2.contiguous()
            y = torch.empty((x2.shape[0], w.shape[0]), dtype=self.output_dtype, device=x2.device)
            _dense.plain_gemm(x2, w, y, bias)
        else:
            y = x2.float() @ w.float().t()
            if bias is not None:
                y = y + bias.float()
            y = y.to(self.output_dtype)
        y = y.reshape(self.bs, ls, self.nh, self.hd)
        W = self.world
        if y.is_cuda:
            res = self._exchange_cuda(y, seq_lens)
        else:
            lq, lk = self.group_heads[0] // W, self.group_heads[1] // W
            parts = (y[:, :, :lq * W], y[:, :, lq * W:(lq + lk) * W], y[:, :, (lq + lk) * W:])
            res = [pre_attn_a2a_varlen_torch(t.contiguous(), self.pg, seq_lens) for t in parts]
        if outputs is not None:
            for dst, src in zip(outputs, res):
                dst.copy_(src)
            return outputs
        return res

    def _forward_cpu(self, x2, w, bias):
        y = x2.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        y = y.to(self.output_dtype)
        if self.comm_op == PreAttnAllToAllCommOp.QKVPackA2A:
            return pre_attn_qkv_pack_a2a_torch(y, self.pg, self.bs, self.local_seq, self.nh, self.hd, self.gqa)
        return pre_attn_a2a_torch(y, self.pg, self.bs, self.local_seq, self.nh, self.hd)

    def _exchange_cuda(self, y: torch.Tensor, seq_lens: Optional[List[int]] = None, group_heads=None,
                       layout: Optional[int] = None, num_ctas: int = 0) -> List[torch.Tensor]:
        """seq -> heads exchange of y [bs, ls, heads, hd] on the strided-exchange kernel: head group g
        of rank d's share lands in d's output buffer at this rank's place in the full sequence.
        Returns views of this rank's outputs, one per head group (valid until the next call)."""
        W, r = self.world, self.rank
        lens = seq_lens if seq_lens is not None else [self.local_seq] * W
        ls, S, off_r = lens[r], sum(lens), sum(lens[:r])
        if S > self.seq:
            raise ValueError("the sequence lengths add up to more than the op was built for")
        groups = group_heads if group_heads is not None else self.group_heads
        layout = self.layout if layout is None else layout
        y = y if y.is_contiguous() else y.contiguous()
        if y.dtype != self.output_dtype:
            raise TypeError("the exchange moves the op's output dtype")
        e = y.element_size()
        nh, hd, bs = y.shape[2], self.hd, self.bs
        copies = [[] for _ in range(W)]
        views, g0, boff = [], 0, 0
        for g, (heads, n) in enumerate(zip(groups, self.out_elems)):
            lh = heads // W
            for d in range(W):
                src = y.data_ptr() + (g0 + d * lh) * hd * e
                if layout == 0:      # [bs, lh, S, hd]
                    dst = self.out_buf.ptr(d, boff) + off_r * hd * e
                    ds = (lh * S * hd * e, hd * e, S * hd * e)
                else:                # [bs, S, lh, hd]
                    dst = self.out_buf.ptr(d, boff) + off_r * lh * hd * e
                    ds = (S * lh * hd * e, lh * hd * e, hd * e)
                copies[d].append((src, dst, (bs, ls, lh), hd * e, (ls * nh * hd * e, nh * hd * e, hd * e), ds))
            shape = (bs, lh, S, hd) if layout == 0 else (bs, S, lh, hd)
            views.append(self.out_buf.view(r, self.output_dtype, shape, boff))
            g0 += heads
            boff += n * _ELEM[self.output_dtype]
        _strided_exchange(self, copies, y.device, num_ctas)
        return views

    # a2a without the GEMM (input already projected)
    def pre_attn_a2a(self, input, seq_lens_cpu=None, num_comm_sm: int = -1, copy_out: bool = True):
        """input [bs, seq/W, heads, hd] (or [bs * seq/W, heads * hd]) -> [bs, heads/W, seq, hd]."""
        if not input.is_cuda:
            return pre_attn_a2a_torch(input, self.pg, self.bs, self.local_seq, self.nh, self.hd)[0]
        lens = _seq_lens_list(seq_lens_cpu, self.world) if seq_lens_cpu is not None else None
        ls = lens[self.rank] if lens is not None else self.local_seq
        out = self._exchange_cuda(input.reshape(self.bs, ls, self.nh, self.hd), lens, [self.nh], 0,
                                  max(num_comm_sm, 0))[0]
        return out.clone() if copy_out else out

    def pre_attn_qkv_pack_a2a(self, qkv, seq_lens_cpu=None, num_comm_sm: int = -1, copy_out: bool = True):
        """qkv [bs, seq/W, heads, hd] with the heads packed q | k | v -> [q, k, v], each
        [bs, seq, heads_x/W, hd]."""
        if not qkv.is_cuda:
            return pre_attn_qkv_pack_a2a_torch(qkv, self.pg, self.bs, self.local_seq, self.nh, self.hd, self.gqa)
        if self.comm_op != PreAttnAllToAllCommOp.QKVPackA2A:
            raise RuntimeError("build the op with comm_op=QKVPackA2A for the packed exchange")
        lens = _seq_lens_list(seq_lens_cpu, self.world) if seq_lens_cpu is not None else None
        ls = lens[self.rank] if lens is not None else self.local_seq
        outs = self._exchange_cuda(qkv.reshape(self.bs, ls, self.nh, self.hd), lens, None, 1, max(num_comm_sm, 0))
        return [o.clone() for o in outs] if copy_out else outs

    def pre_attn_a2a_no_cpy(self, input, seq_lens_cpu=None, num_comm_sm: int = -1, comm_buf_idx: int = 0):
        """Same, returning views of the op's symmetric output buffer (valid until the next call)."""
        return self.pre_attn_a2a(input, seq_lens_cpu, num_comm_sm, copy_out=False)

    def pre_attn_qkv_pack_a2a_no_cpy(self, qkv, seq_lens_cpu=None, num_comm_sm: int = -1, comm_buf_idx: int = 0):
        return self.pre_attn_qkv_pack_a2a(qkv, seq_lens_cpu, num_comm_sm, copy_out=False)

    def get_input_comm_buf(self, input, comm_buf_idx: int = 0):
        return input

    def sp_group_barrier_all(self) -> None:
        dist.barrier(group=self.pg)

    def profiling(self, input, weight, bias=None, input_scale=None, weight_scale=None, output_scale=None,
                  fast_accum=False, num_comm_sm=-1, sm_margin=0, prof_ctx=None):
        from ..tuning.profiling import profile_call
        w = as_nk(weight, self.transpose_weight)
        return profile_call(self, "gemm_a2a_transpose", lambda: self.forward(input, weight, bias=bias), prof_ctx,
                            key=(self.bs * self.local_seq, w.shape[0], self.hidden))


class AllToAllTransposeGemm(FusedOpBase):
    def __init__(self, tp_group, nnodes: int, sp_size: int, bs: int, num_head: int, seq: int, head_dim: int,
                 input_dtype: torch.dtype, output_dtype: Optional[torch.dtype] = None,
                 max_num_comm_buf: int = 1, a2a_only: bool = False, timeout_s: Optional[float] = None):
        super().__init__(_sp_group(tp_group, sp_size), nnodes, timeout_s)
        W = self.world
        if seq % W or num_head % W:
            raise ValueError("seq and num_head must divide over the group")
        self.bs, self.nh, self.seq, self.hd = bs, num_head, seq, head_dim
        self.local_seq, self.local_nh = seq // W, num_head // W
        self.hidden = num_head * head_dim
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.a2a_only = a2a_only
        self.land = SymmBuffer(bs * self.local_seq * self.hidden * _ELEM[input_dtype], self.pg)

    def forward(self, input: torch.Tensor, weight: torch.Tensor, seq_lens_cpu=None,
                bias: Optional[torch.Tensor] = None, output: Optional[torch.Tensor] = None,
                input_scale=None, weight_scale=None, output_scale=None, fast_accum: bool = False,
                transpose_weight: bool = False, all_to_all_option=None,
                a2a_transpose_output: Optional[torch.Tensor] = None, num_comm_sm: int = -1,
                sm_margin: int = 0) -> torch.Tensor:
        """input [bs, heads/W, seq, hd] (``a2a_only``: [bs, seq, heads/W, hd]) -> [bs, seq/W, N]."""
        if seq_lens_cpu is not None:
            # ranks with different sequence lengths: the strided exchange, then the GEMM kernel
            gi = self.post_attn_a2a(input, seq_lens_cpu, copy_out=False)
            if a2a_transpose_output is not None:
                a2a_transpose_output.copy_(gi.reshape(a2a_transpose_output.shape))
            res = self.gemm_only(gi, weight, bias=bias, output=output, transpose_weight=transpose_weight)
            return res if output is not None else res.reshape(self.bs, gi.shape[1], -1)
        w = as_nk(weight, transpose_weight)
        N = w.shape[0]
        M = self.bs * self.local_seq
        self._begin_call()
        if not input.is_cuda:
            gi = post_attn_a2a_torch(input, self.pg, self.a2a_only)
            y = gi.reshape(M, self.hidden).float() @ w.float().t()
            if bias is not None:
                y = y + bias.float()
            res = y.to(self.output_dtype).reshape(self.bs, self.local_seq, N)
            if a2a_transpose_output is not None:
                a2a_transpose_output.copy_(gi.reshape(a2a_transpose_output.shape))
        else:
            x = input if input.is_contiguous() else input.contiguous()
            res = torch.empty((self.bs, self.local_seq, N), dtype=self.output_dtype, device=input.device)
            keep: list = []
            land_local = self.land.view(self.rank, self.input_dtype, (M, self.hidden))
            args = A2AArgs()
            base = _dense.base_args(land_local, w, bias, self.output_dtype, m=M, status=self.status, keep=keep)
            base.M = M
            base.d, base.ldd = res.data_ptr(), N
            base.num_sms = self._num_sms(sm_margin)   # (the push runs in the GEMM's own CTAs)
            base.mode, base.rank, base.world = 4, self.rank, self.world
            base.epoch, base.timeout_ns = self.epoch, int(self.timeout_s * 1e9)
            base.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
            for r in range(self.world):
                base.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
                args.a2a_flags[r] = self.ctrl.ptr(r, OFF_CTR)
                args.land[r] = self.land.ptr(r)
            args.base = base
            args.bs, args.local_seq, args.hd = self.bs, self.local_seq, self.hd
            args.layout = 1 if self.a2a_only else 0
            args.attn = x.data_ptr()
            args.copy_local = 1 if a2a_transpose_output is not None else 0
            _native.check(_native.lib().fluxb_ulysses_gemm(ctypes.byref(args)), "fluxb_ulysses_gemm")
            self._after_launch()
            if a2a_transpose_output is not None:
                # the landing buffer holds one slab per source rank in the source's own layout
                W, lh = self.world, self.local_nh
                if self.a2a_only:
                    gi = self.land.view(self.rank, self.input_dtype, (W, M, lh, self.hd)).permute(1, 0, 2, 3)
                else:
                    gi = self.land.view(self.rank, self.input_dtype, (W, lh, M, self.hd)).permute(2, 0, 1, 3)
                a2a_transpose_output.copy_(gi.reshape(a2a_transpose_output.shape))
        if output is not None:
            output.copy_(res.reshape(output.shape))
            return output
        return res

    __call__ = forward

    def post_attn_a2a(self, input, seq_lens_cpu=None, all_to_all_option=None, num_comm_sm: int = -1,
                      copy_out: bool = True):
        """heads -> seq exchange alone: input [bs, heads/W, seq, hd] (``a2a_only``: [bs, seq, heads/W,
        hd]) -> [bs, seq/W (this rank's length), heads * hd], heads ordered by source rank."""
        lens = _seq_lens_list(seq_lens_cpu, self.world) if seq_lens_cpu is not None else None
        if not input.is_cuda:
            if lens is not None:
                return post_attn_a2a_varlen_torch(input, self.pg, self.a2a_only, lens)
            return post_attn_a2a_torch(input, self.pg, self.a2a_only)
        W, r = self.world, self.rank
        lens = lens if lens is not None else [self.local_seq] * W
        S = sum(lens)
        x = input if input.is_contiguous() else input.contiguous()
        e, hd, lh, nh, bs = x.element_size(), self.hd, self.local_nh, self.nh, self.bs
        need = bs * max(lens) * self.hidden * e
        if need > self.land.nbytes:          # every rank sees the same lengths: a collective re-allocation
            self.land = SymmBuffer(need, self.pg)
        copies = [[] for _ in range(W)]
        for d in range(W):
            off_d, ls_d = sum(lens[:d]), lens[d]
            if self.a2a_only:                # [bs, S, lh, hd]
                src = x.data_ptr() + off_d * lh * hd * e
                ss = (S * lh * hd * e, lh * hd * e, hd * e)
            else:                            # [bs, lh, S, hd]
                src = x.data_ptr() + off_d * hd * e
                ss = (lh * S * hd * e, hd * e, S * hd * e)
            dst = self.land.ptr(d) + r * lh * hd * e
            copies[d].append((src, dst, (bs, ls_d, lh), hd * e, ss, (ls_d * nh * hd * e, nh * hd * e, hd * e)))
        _strided_exchange(self, copies, x.device, max(num_comm_sm, 0))
        out = self.land.view(r, self.input_dtype, (bs, lens[r], self.hidden))
        return out.clone() if copy_out else out

    def post_attn_a2a_no_cpy(self, input, seq_lens_cpu=None, all_to_all_option=None, num_comm_sm: int = -1,
                             comm_buf_idx: int = 0):
        """Same, returning a view of the op's symmetric buffer (valid until the next call)."""
        return self.post_attn_a2a(input, seq_lens_cpu, copy_out=False)

    def gemm_only(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, transpose_weight=False):
        w = as_nk(weight, transpose_weight)
        x2 = input.reshape(-1, input.shape[-1])
        out = output if output is not None else torch.empty(
            (x2.shape[0], w.shape[0]), dtype=self.output_dtype, device=input.device)
        if not input.is_cuda:
            y = x2.float() @ w.float().t()
            if bias is not None:
                y = y + bias.float()
            out.copy_(y.to(self.output_dtype).reshape(out.shape))
            return out
        return _dense.plain_gemm(x2 if x2.is_contiguous() else x2.contiguous(), w, out.view(x2.shape[0], -1), bias)

    def sp_group_barrier_all(self) -> None:
        dist.barrier(group=self.pg)

    def reset_signals(self) -> None:
        """Reference API; nothing to reset here: flags carry the call number."""

    def profiling(self, input, weight, bias=None, output=None, prof_ctx=None, **kw):
        from ..tuning.profiling import profile_call
        w = as_nk(weight, kw.get("transpose_weight", False))
        return profile_call(self, "a2a_transpose_gemm", lambda: self.forward(input, weight, bias=bias), prof_ctx,
                            key=(self.bs * self.local_seq, w.shape[0], self.hidden))
