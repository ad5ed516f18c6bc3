"""``BlockScaleGemm``: FP8 (e4m3) GEMM with 1x128 activation scales and 128x128 weight scales,
fp32 promotion of every 128-deep k-block (reference: ``flux.BlockScaleGemm``,
``src/pybind/gemm_only.cc:77-170``, ``src/comm_none/ths_op/blockscale_gemm.cc``).

``out = sum_kb (A_q[:, kb] @ B_q[:, kb]^T) * sA[row-block, kb, row] * sB[col-block, kb]``

with ``sA [M/128, K/128, 128]`` and ``sB [N/128, K/128]`` holding the *inverse* scales written
by ``Quantization``. ``blockscale_gemm_torch`` states the same math in PyTorch (the oracle of
``test/python/gemm_only/test_blockwise_scale_gemm_only.py:200-261``)."""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from . import _dense

BLOCK = 128


def blockscale_gemm_torch(a_q: torch.Tensor, b_q: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor,
                          out_dtype: torch.dtype = torch.bfloat16, bias: Optional[torch.Tensor] = None
                          ) -> torch.Tensor:
    """a_q [M,K], b_q [N,K] fp8; sa [ceil(M/128), K/128, 128]; sb [N/128, K/128] or, for
    per-column ("groupwise") weight scales, [N/128, K/128, 128]."""
    M, K = a_q.shape
    N = b_q.shape[0]
    KB = K // BLOCK
    a = a_q.float().view(M, KB, BLOCK)
    b = b_q.float().view(N, KB, BLOCK)
    sa_rows = sa.permute(0, 2, 1).reshape(-1, KB)[:M]                       # [M, KB]
    if sb.dim() == 2:
        sb_rows = sb.repeat_interleave(BLOCK, dim=0)[:N]                    # [N, KB]
    else:
        sb_rows = sb.permute(0, 2, 1).reshape(-1, KB)[:N]
    acc = torch.einsum("mkc,nkc->kmn", a, b)                                # per-k-block products
    acc = acc * sa_rows.t()[:, :, None] * sb_rows.t()[:, None, :]
    out = acc.sum(0)
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)


def blockscale_args(a, w, sa, sb, bias, out_dtype, m, status=None, keep=None) -> _dense.DenseArgs:
    if a.dtype != torch.float8_e4m3fn or w.dtype != torch.float8_e4m3fn:
        raise TypeError("block-scaled GEMM takes float8_e4m3fn operands")
    K, N = a.shape[1], w.shape[0]
    if K % BLOCK or N % BLOCK:
        raise ValueError("K and N must be multiples of 128")
    if sa.dtype != torch.float32 or sb.dtype != torch.float32 or not sa.is_contiguous() or not sb.is_contiguous():
        raise TypeError("scales must be contiguous float32 tensors")
    if sa.dim() != 3 or sa.shape[1] != K // BLOCK or sa.shape[2] != BLOCK or sa.shape[0] < -(-a.shape[0] // BLOCK):
        raise ValueError(f"input_scale must be [ceil(rows/128), {K // BLOCK}, 128], got {tuple(sa.shape)}")
    groupwise = sb.dim() == 3
    if tuple(sb.shape) not in ((N // BLOCK, K // BLOCK), (N // BLOCK, K // BLOCK, BLOCK)):
        raise ValueError(f"weight_scale must be [{N // BLOCK}, {K // BLOCK}] or, one per weight row, "
                         f"[{N // BLOCK}, {K // BLOCK}, {BLOCK}]; got {tuple(sb.shape)}")
    # single CTAs on 128 x 256 tiles where N allows (FLUXB_BS_TILE_N=128 pins 128 x 128); FLUXB_BS_CTA_GROUP=2
    # asks for CTA pairs on 256 x 128 tiles (measured slower)
    cta_group = int(os.environ.get("FLUXB_BS_CTA_GROUP", "1"))
    tile_n = int(os.environ.get("FLUXB_BS_TILE_N", "128" if cta_group == 2 else "0"))
    args = _dense.base_args(a, w, bias, out_dtype, tile_n=tile_n, cta_group=cta_group, m=m, status=status, keep=keep)
    args.sa, args.sb = sa.data_ptr(), sb.data_ptr()
    args.blockscale = 2 if groupwise else 1
    return args


class BlockScaleGemm:
    def __init__(self, input_dtype: torch.dtype = torch.float8_e4m3fn,
                 weight_dtype: torch.dtype = torch.float8_e4m3fn,
                 output_dtype: Optional[torch.dtype] = None, num_streams: int = 2):
        if input_dtype != torch.float8_e4m3fn or weight_dtype != torch.float8_e4m3fn:
            raise TypeError("BlockScaleGemm supports float8_e4m3fn inputs")
        self.input_dtype, self.weight_dtype = input_dtype, weight_dtype
        self.output_dtype = output_dtype or torch.bfloat16
        # side streams of the per-expert forms: an expert with fewer tiles than the GPU has SMs leaves the
        # rest to the next expert's launch
        self.num_streams = max(1, int(num_streams))
        self._streams: list = []

    def forward(self, input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                output: Optional[torch.Tensor] = None, input_scale: Optional[torch.Tensor] = None,
                weight_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        if input_scale is None or weight_scale is None:
            raise ValueError("block-scaled GEMM needs input_scale and weight_scale")
        M, N = input.shape[0], weight.shape[0]
        if not input.is_cuda:
            # CPU tensors go through the PyTorch statement of the op
            res = blockscale_gemm_torch(input, weight, input_scale, weight_scale, self.output_dtype, bias)
            if output is not None:
                output.copy_(res)
                return output
            return res
        out = output if output is not None else torch.empty((M, N), dtype=self.output_dtype, device=input.device)
        keep: list = []
        args = blockscale_args(input, weight, input_scale, weight_scale, bias, self.output_dtype, M, keep=keep)
        args.M = M
        args.d, args.ldd = out.data_ptr(), out.stride(0)
        args.mode, args.rank, args.world, args.epoch = _dense.PLAIN, 0, 1, 1
        _dense.run(args)
        return out

    __call__ = forward

    def wgrad(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None):
        """Weight-gradient form: both operands carry 1x128 scales (``weight_scale`` is
        [N/128, K/128, 128])."""
        return self.forward(input, weight, bias, output, input_scale, weight_scale)

    def _per_expert(self, input, input_splits: Sequence[int], weight, bias, output, input_scale, weight_scale):
        M, N = input.shape[0], weight.shape[1]
        out = output if output is not None else torch.empty((M, N), dtype=self.output_dtype, device=input.device)
        # (splits normally live on the host, as in the reference; a device tensor costs one sync here)
        splits = [int(v) for v in (input_splits.tolist() if torch.is_tensor(input_splits) else input_splits)]
        jobs, row = [], 0
        for e, cnt in enumerate(splits):
            if cnt:
                if row % BLOCK:
                    raise ValueError("expert row ranges must start on multiples of 128 (1x128 scale blocks)")
                jobs.append((e, row, cnt))
            row += cnt

        def run(e, row, cnt):
            sa_e = input_scale[row // BLOCK:(row + cnt + BLOCK - 1) // BLOCK]
            self.forward(input[row:row + cnt], weight[e], None if bias is None else bias[e],
                         out[row:row + cnt], sa_e, weight_scale[e])

        n = min(self.num_streams, len(jobs))
        if n <= 1 or not input.is_cuda:
            for j in jobs:
                run(*j)
            return out
        # fork: every side stream starts after what the caller's stream has queued so far; join: the
        # caller's stream continues after all of them
        cur = torch.cuda.current_stream(input.device)
        while len(self._streams) < n:
            self._streams.append(torch.cuda.Stream(input.device))
        fork = torch.cuda.Event()
        fork.record(cur)
        for i in range(n):
            self._streams[i].wait_event(fork)
        for i, j in enumerate(jobs):
            with torch.cuda.stream(self._streams[i % n]):
                run(*j)
        for i in range(n):
            done = torch.cuda.Event()
            done.record(self._streams[i])
            cur.wait_event(done)
        return out

    def forward_multistream(self, input, input_splits, weight, bias=None, output=None, input_scale=None,
                            weight_scale=None):
        """Per-expert block-scaled GEMMs: ``weight [E, N, K]``, ``weight_scale [E, N/128, K/128]``,
        rows of ``input`` grouped by expert as given by ``input_splits`` (host values, as in the
        reference). One launch per expert, dealt over ``num_streams`` side streams (reference:
        ``forward_multi_stream``, python/flux/cpp_mod.pyi:283-292)."""
        return self._per_expert(input, input_splits, weight, bias, output, input_scale, weight_scale)

    wgrad_multistream = forward_multistream
    forward_multi_stream = forward_multistream   # spelling of the reference's stub file
    forward_grouped = forward_multistream
    wgrad_grouped = forward_multistream

    def reference(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None,
                  is_groupwise_b: bool = False):
        res = blockscale_gemm_torch(input, weight, input_scale, weight_scale, self.output_dtype, bias)
        if output is not None:
            output.copy_(res)
            return output
        return res

    def profiling(self, input, weight, bias=None, output=None, input_scale=None, weight_scale=None, prof_ctx=None):
        from ..tuning.profiling import profile_call
        return profile_call(self, "blockscale_gemm",
                            lambda: self.forward(input, weight, bias, output, input_scale, weight_scale), prof_ctx)
