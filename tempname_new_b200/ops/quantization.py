"""``Quantization``: block-scaled FP8 quantisation, 1x128 and 128x128, with optional transposed
output (reference: ``flux.Quantization``, ``src/pybind/quantization.cc:30-57``,
``src/quantization/ths_op/quantization.cc``). Layouts are documented in
``csrc/aux/quantize.cu``; ``quantize_*_torch`` below state the same math in PyTorch and serve
as the CPU path and as the test oracle."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _native
from ._dense import current_stream_ptr, dtype_code

BLOCK = 128
_FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}
Quad = Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]


def _scale_of(amax: torch.Tensor, eps: float, fp8_max: float) -> torch.Tensor:
    a = torch.clamp(amax, min=eps)
    # tensor / tensor is a true division (scalar / tensor would go through a reciprocal)
    s = torch.where(a == 0, torch.ones_like(a),
                    torch.full_like(a, fp8_max) / torch.where(a == 0, torch.ones_like(a), a))
    return torch.where(torch.isinf(s), torch.full_like(s, 3.3895313892515355e38), s)


def _pad_blocks(x: torch.Tensor) -> torch.Tensor:
    M, K = x.shape[-2:]
    pm, pk = (-M) % BLOCK, (-K) % BLOCK
    return torch.nn.functional.pad(x, (0, pk, 0, pm)) if (pm or pk) else x


def quantize_vector_blockwise_torch(x: torch.Tensor, out_dtype=torch.float8_e4m3fn, eps: float = 0.0):
    """1x128 blocks along the last dim: returns (q [M,K], scale_inv [M/128, K/128, 128])."""
    M, K = x.shape
    xp = _pad_blocks(x.float())
    MB, KB = xp.shape[0] // BLOCK, xp.shape[1] // BLOCK
    blocks = xp.view(MB, BLOCK, KB, BLOCK)
    scale = _scale_of(blocks.abs().amax(dim=3), eps, _FP8_MAX[out_dtype])       # [MB, 128, KB]
    q = (blocks * scale.unsqueeze(3)).clamp(-_FP8_MAX[out_dtype], _FP8_MAX[out_dtype])
    q = q.reshape(MB * BLOCK, KB * BLOCK)[:M, :K].to(out_dtype)
    return q, (1.0 / scale).permute(0, 2, 1).contiguous()


def quantize_square_blockwise_torch(x: torch.Tensor, out_dtype=torch.float8_e4m3fn, eps: float = 0.0):
    """128x128 blocks: returns (q [M,K], scale_inv [M/128, K/128])."""
    M, K = x.shape
    xp = _pad_blocks(x.float())
    MB, KB = xp.shape[0] // BLOCK, xp.shape[1] // BLOCK
    blocks = xp.view(MB, BLOCK, KB, BLOCK)
    scale = _scale_of(blocks.abs().amax(dim=(1, 3)), eps, _FP8_MAX[out_dtype])  # [MB, KB]
    q = (blocks * scale[:, None, :, None]).clamp(-_FP8_MAX[out_dtype], _FP8_MAX[out_dtype])
    q = q.reshape(MB * BLOCK, KB * BLOCK)[:M, :K].to(out_dtype)
    return q, 1.0 / scale


class Quantization:
    def __init__(self, input_dtype: torch.dtype, output_dtype: torch.dtype, num_streams: int = 2):
        if input_dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise TypeError("input must be bf16, fp16 or fp32")
        if output_dtype not in _FP8_MAX:
            raise TypeError("output must be float8_e4m3fn or float8_e5m2")
        self.input_dtype, self.output_dtype = input_dtype, output_dtype
        self.num_streams = num_streams  # the batched kernel covers all matrices in one launch

    # ------------------------------------------------------------------------------
    def _run(self, x: torch.Tensor, square: bool, transpose: bool, eps: float) -> Quad:
        batched = x.dim() == 3
        if x.dtype != self.input_dtype:
            raise TypeError(f"expected {self.input_dtype}, got {x.dtype}")
        x = x if x.stride(-1) == 1 and (not batched or x.is_contiguous()) else x.contiguous()
        B = x.shape[0] if batched else 1
        M, K = x.shape[-2:]
        MB, KB = -(-M // BLOCK), -(-K // BLOCK)
        lead = (B,) if batched else ()
        if not x.is_cuda:
            return self._run_torch(x, square, transpose, eps)
        dev = x.device
        q = torch.empty(lead + (M, K), dtype=self.output_dtype, device=dev)
        s_shape = (MB, KB) if square else (MB, KB, BLOCK)
        st_shape = (KB, MB) if square else (KB, MB, BLOCK)
        s = torch.empty(lead + s_shape, dtype=torch.float32, device=dev)
        qt = torch.empty(lead + (K, M), dtype=self.output_dtype, device=dev) if transpose else None
        s_t = torch.empty(lead + st_shape, dtype=torch.float32, device=dev) if transpose else None
        rc = _native.lib().fluxb_quantize_blockwise(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_int64(x.stride(-2)), dtype_code(x.dtype),
            ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(qt.data_ptr() if transpose else None),
            ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(s_t.data_ptr() if transpose else None),
            M, K, B, int(square), ctypes.c_float(eps), dtype_code(self.output_dtype),
            ctypes.c_void_p(current_stream_ptr(dev)))
        _native.check(rc, "fluxb_quantize_blockwise")
        return q, s, qt, s_t

    def _run_torch(self, x, square, transpose, eps) -> Quad:
        fn = quantize_square_blockwise_torch if square else quantize_vector_blockwise_torch
        if x.dim() == 3:
            outs = [self._run_torch(m, square, transpose, eps) for m in x]
            stack = lambda i: torch.stack([o[i] for o in outs]) if outs[0][i] is not None else None  # noqa: E731
            return stack(0), stack(1), stack(2), stack(3)
        q, s = fn(x, self.output_dtype, eps)
        if not transpose:
            return q, s, None, None
        if square:
            return q, s, q.t().contiguous(), s.t().contiguous()
        qt, s_t = fn(x.t().contiguous(), self.output_dtype, eps)
        return q, s, qt, s_t

    def quantize_vector_blockwise(self, input: torch.Tensor, return_transpose: bool = True, eps: float = 0.0) -> Quad:
        return self._run(input, False, return_transpose, eps)

    def quantize_square_blockwise(self, input: torch.Tensor, return_transpose: bool = True, eps: float = 0.0) -> Quad:
        return self._run(input, True, return_transpose, eps)

    def batch_quantize_square_blockwise(self, input: torch.Tensor, return_transpose: bool = True, eps: float = 0.0) -> Quad:
        if input.dim() != 3:
            raise ValueError("input must have 3 dimensions")
        return self._run(input, True, return_transpose, eps)
