"""``AGKernel``: all-gather fused with GEMM (column-parallel linear forward).

``out[M, N/W] = all_gather_M(input[M/W, K]) @ weight[N/W, K]^T (+bias)``

On CUDA one persistent tcgen05 kernel does both: two warps of every CTA push this rank's
shard into the peers' landing buffers through a ring of bulk copies (global -> shared ->
peer global, first to the peer that will consume it first) and publish an arrival flag per
shard unit, while the TMA producer of the same kernel starts on the local shard and gates
each remote M-tile on its unit's flag.
Reference: ``flux.AGKernel`` (``src/pybind/ag_gemm.cc:28-106``,
``src/ag_gemm/ths_op/all_gather_gemm_op.cc``, ``src/coll/ths_op/all_gather_op.cc``): copy
engine pulls on a side stream plus a flag-gated GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _dense
from ._fused_base import MAX_FLAG_WORDS, OFF_CTR, OFF_LOCAL, OFF_START, FusedOpBase
from .gemm_only import _out_dtype, apply_act, as_nk
from .options import AllGatherOption
from ..parallel.symm import SymmBuffer, _ELEM


class AGKernel(FusedOpBase):
    def __init__(self, tp_group, nnodes: int, full_m: int, n_dim: int, k_dim: int,
                 input_dtype: torch.dtype, output_dtype: Optional[torch.dtype] = None,
                 use_pdl: bool = False, timeout_s: Optional[float] = None):
        super().__init__(tp_group, nnodes, timeout_s)
        self.full_m, self.n_dim, self.k_dim = full_m, n_dim, k_dim
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.use_pdl = use_pdl
        if full_m % self.world != 0:
            raise ValueError("full_m must be a multiple of the world size")
        if (full_m + 127) // 128 + 8 > MAX_FLAG_WORDS:
            raise ValueError("full_m too large for the flag block")
        self.land = SymmBuffer(full_m * k_dim * _ELEM[input_dtype], self.pg) if self.world > 1 else None
        self.scale_land = None  # allocated at the first block-scaled call

    def forward(self, input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                output: Optional[torch.Tensor] = None, input_scale: Optional[torch.Tensor] = None,
                weight_scale: Optional[torch.Tensor] = None, output_scale: Optional[torch.Tensor] = None,
                fast_accum: bool = False, transpose_weight: bool = False,
                all_gather_option: Optional[AllGatherOption] = None,
                gathered_input: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
        """``act`` (not in the reference API) fuses gelu / relu / silu after the bias."""
        w = as_nk(weight, transpose_weight)
        seg, K = input.shape
        M, N = seg * self.world, w.shape[0]
        if M > self.full_m or K != self.k_dim:
            raise ValueError(f"AGKernel was built for M <= {self.full_m}, K = {self.k_dim}; got M={M}, K={K}")
        self._begin_call()
        if not input.is_cuda:
            if input_scale is not None and input_scale.dim() == 3:
                raise NotImplementedError("block-scaled AG+GEMM has no CPU path")
            return self._forward_cpu(input, w, bias, output, input_scale, weight_scale, gathered_input, act)
        a = input if input.is_contiguous() else input.contiguous()
        out = output if output is not None else torch.empty((M, N), dtype=self.output_dtype, device=input.device)
        keep: list = []
        blockscale = input_scale is not None and input_scale.dim() == 3
        if blockscale:
            # fp8 payload and its 1x128 scales travel together; scales land in their own buffer
            from .blockscale_gemm import blockscale_args
            if seg % 128:
                raise ValueError("block-scaled AG+GEMM needs M/W to be a multiple of 128")
            args = blockscale_args(a, w, input_scale, weight_scale, bias, self.output_dtype, M,
                                   status=self.status, keep=keep)
            args.act = _dense.ACT[act]
            if self.world > 1:
                if self.scale_land is None:
                    self.scale_land = SymmBuffer(self.full_m // 128 * (self.k_dim // 128) * 512, self.pg)
                for r in range(self.world):
                    args.ag_scale_land[r] = self.scale_land.ptr(r)
        else:
            if input_scale is not None and input_scale.numel() > 1:
                # one scale per input row ([M/W, 1], the reference's int8 convention): the GEMM needs
                # the scales of all M rows, so they are gathered too (a small launch of the row-exchange kernel)
                input_scale = self._gather_row_scales(input_scale, seg)
            args = _dense.base_args(a, w, bias, self.output_dtype, input_scale, weight_scale,
                                    act=act, m=M, status=self.status, keep=keep)
        args.M = M
        args.d, args.ldd = out.data_ptr(), out.stride(0)
        args.mode, args.rank, args.world = _dense.ALLGATHER, self.rank, self.world
        args.epoch = self.epoch
        args.timeout_ns = int(self.timeout_s * 1e9)
        if self.world > 1:
            for r in range(self.world):
                args.ag_land[r] = self.land.ptr(r)
                args.ag_flags[r] = self.ctrl.ptr(r, OFF_CTR)
                args.start_ctr[r] = self.ctrl.ptr(r, OFF_START)
            args.local_cnt = self.ctrl.ptr(self.rank, OFF_LOCAL)
        args.num_sms = self._num_sms()
        _dense.run(args)
        if gathered_input is not None:
            self._copy_gathered(a, gathered_input, seg, K)
        self._after_launch()
        return out

    __call__ = forward

    def _gather_row_scales(self, scale: torch.Tensor, seg: int) -> torch.Tensor:
        """[M/W] per-row scales of every rank -> [M] in rank order."""
        if scale.numel() != seg:
            raise ValueError(f"input_scale must hold 1 or {seg} (rows of this rank's shard) values")
        s = scale.reshape(-1).float().contiguous()
        if self.world == 1:
            return s
        if not s.is_cuda:
            parts = [torch.empty_like(s) for _ in range(self.world)]
            torch.distributed.all_gather(parts, s, group=self.pg)
            return torch.cat(parts)
        from .coll import AllGatherOp
        rows = (seg + 3) // 4                       # rows of four floats (16 bytes)
        if getattr(self, "_scale_ag", None) is None or self._scale_ag.max_rows < rows * self.world:
            self._scale_ag = AllGatherOp(self.pg, 1, rows * self.world, 4, torch.float32)
        padded = torch.zeros(rows * 4, dtype=torch.float32, device=s.device)
        padded[:seg] = s
        got = self._scale_ag.run(padded.view(rows, 4)).reshape(self.world, rows * 4)
        return got[:, :seg].reshape(-1).contiguous()

    def _copy_gathered(self, a, gathered_input, seg, K):
        if self.world == 1:
            gathered_input.copy_(a)
            return
        land = self.land.view(self.rank, self.input_dtype, (self.world, seg, K))
        g = gathered_input.view(self.world, seg, K)
        g.copy_(land)
        g[self.rank].copy_(a)

    def gemm_only(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, transpose_weight=False):
        """GEMM on an already gathered ``input[M, K]`` (no communication)."""
        w = as_nk(weight, transpose_weight)
        out = output if output is not None else torch.empty(
            (input.shape[0], w.shape[0]), dtype=self.output_dtype, device=input.device)
        if not input.is_cuda:
            out.copy_((input.float() @ w.float().t()).to(self.output_dtype))
            return out
        return _dense.plain_gemm(input, w, out, bias, input_scale, weight_scale)

    def profiling(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, transpose_weight=False, all_gather_option=None,
                  gathered_input=None, prof_ctx=None):
        from ..tuning.profiling import profile_call
        w = as_nk(weight, transpose_weight)
        blockscaled = input_scale is not None and input_scale.dim() == 3     # fixed tile shape: nothing to sweep
        key = None if blockscaled else (input.shape[0] * self.world, w.shape[0], input.shape[1])
        return profile_call(self, "ag_gemm", lambda: self.forward(
            input, weight, bias, output, input_scale, weight_scale, transpose_weight=transpose_weight), prof_ctx,
            key=key, segmented_rows=input.shape[0])

    def _forward_cpu(self, a, w, bias, output, sa, sb, gathered_input, act=None):
        W, r = self.world, self.rank
        seg, K = a.shape
        if W > 1:
            self._cpu_start_handshake()
            for d in range(1, W):
                peer = (r - d) % W
                self.land.view(peer, self.input_dtype, (W, seg, K))[r].copy_(a)
                self._cpu_words(peer, OFF_CTR, 8)[r] = self.epoch
            mine_flags = self._cpu_words(r, OFF_CTR, 8)
            mine_flags[r] = self.epoch
            self._cpu_wait(mine_flags[:W], self.epoch, "all-gather arrivals")
            full = self.land.view(r, self.input_dtype, (W, seg, K)).clone()
            full[r].copy_(a)
            full = full.view(W * seg, K)
        else:
            full = a
        acc = full.float() @ w.float().t()
        if sa is not None:
            if sa.numel() > 1:
                sa = self._gather_row_scales(sa, seg).reshape(-1, 1)
            acc = acc * sa.float()
        if sb is not None:
            _dense.check_scale(sb, w.shape[0], "weight_scale")
            acc = acc * (sb.float().reshape(1, -1) if sb.numel() > 1 else sb.float())
        if bias is not None:
            acc = acc + bias.float()
        acc = apply_act(acc, act)
        res = acc.to(self.output_dtype)
        if gathered_input is not None:
            gathered_input.copy_(full)
        if output is not None:
            output.copy_(res)
            return output
        return res
