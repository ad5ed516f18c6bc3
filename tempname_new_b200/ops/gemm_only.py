"""``GemmOnly``: plain GEMM on the sm_100a tcgen05 kernel (reference: ``flux.GemmOnly``,
``src/pybind/gemm_only.cc:35-75``, ``src/comm_none/ths_op/gemm_only.cc``)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _dense

_IN_DTYPES = (torch.bfloat16, torch.float16, torch.float8_e4m3fn, torch.float8_e5m2, torch.int8)


def _out_dtype(input_dtype: torch.dtype, output_dtype: Optional[torch.dtype]) -> torch.dtype:
    if output_dtype is not None:
        return output_dtype
    return torch.bfloat16 if input_dtype in (torch.float8_e4m3fn, torch.float8_e5m2, torch.int8) else input_dtype


def as_nk(weight: torch.Tensor, transpose_weight: bool) -> torch.Tensor:
    """The kernels take B as [N, K]. K contiguous is the native form; 16-bit weights held as [K, N]
    (``transpose_weight``, or a transposed view passed without it) are read in place as MN-major
    operand tiles on the GPU. Anything else (8-bit [K, N] weights, odd pitches, CPU tensors' views are
    fine as they are) is re-laid out once per call."""
    from ._dense import kn_in_place
    w = weight.t() if transpose_weight else weight
    if w.stride(-1) == 1 or (w.is_cuda and kn_in_place(w)):
        return w
    return w.contiguous()


def apply_act(x: torch.Tensor, act: Optional[str]) -> torch.Tensor:
    """Torch statement of the epilogue activations of the dense kernel."""
    if act in (None, "none"):
        return x
    if act in ("gelu", "gelu_tanh"):
        return torch.nn.functional.gelu(x, approximate="tanh")
    if act == "relu":
        return torch.relu(x)
    if act == "silu":
        return torch.nn.functional.silu(x)
    raise ValueError(f"unknown activation {act}")


class GemmOnly:
    def __init__(self, input_dtype: torch.dtype, weight_dtype: Optional[torch.dtype] = None,
                 output_dtype: Optional[torch.dtype] = None, transpose_weight: bool = False,
                 use_fp8_gemm: bool = False):
        weight_dtype = weight_dtype or input_dtype
        # float32 is accepted for the CPU (test) path only; the GPU kernels take 16- and 8-bit inputs
        if input_dtype not in _IN_DTYPES + (torch.float32,) or weight_dtype != input_dtype:
            raise TypeError(f"GemmOnly supports {_IN_DTYPES} with matching weight dtype")
        self.input_dtype = input_dtype
        self.output_dtype = _out_dtype(input_dtype, output_dtype)
        self.transpose_weight = transpose_weight
        self.use_fp8_gemm = use_fp8_gemm

    def forward(self, input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                output_buf: Optional[torch.Tensor] = None, input_scale: Optional[torch.Tensor] = None,
                weight_scale: Optional[torch.Tensor] = None, output_scale: Optional[torch.Tensor] = None,
                fast_accum: bool = False) -> torch.Tensor:
        w = as_nk(weight, self.transpose_weight)
        M, N = input.shape[0], w.shape[0]
        if not input.is_cuda:
            return self._forward_cpu(input, w, bias, output_buf, input_scale, weight_scale)
        out = output_buf if output_buf is not None else torch.empty(
            (M, N), dtype=self.output_dtype, device=input.device)
        a = input if input.stride(-1) == 1 else input.contiguous()
        _dense.plain_gemm(a, w, out, bias, input_scale, weight_scale)
        return out

    def _forward_cpu(self, a, w, bias, out, sa, sb):
        acc = a.float() @ w.float().t()
        if sa is not None:
            vec = _dense.check_scale(sa, a.shape[0], "input_scale")
            acc = acc * (sa.float().reshape(-1, 1) if vec else sa.float().reshape(-1)[0])
        if sb is not None:
            vec = _dense.check_scale(sb, w.shape[0], "weight_scale")
            acc = acc * (sb.float().reshape(1, -1) if vec else sb.float().reshape(-1)[0])
        if bias is not None:
            acc = acc + bias.float()
        res = acc.to(self.output_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def profiling(self, input, weight, bias=None, output_buf=None, input_scale=None, weight_scale=None,
                  output_scale=None, fast_accum=False, prof_ctx=None):
        from ..tuning.profiling import profile_dense_plain
        return profile_dense_plain(self, input, weight, bias, output_buf, input_scale, weight_scale, prof_ctx)

    __call__ = forward
