"""ctypes view of ``fluxb_dense_gemm`` (csrc/include/fluxb.h) shared by GemmOnly, AGKernel and
GemmRS."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from .. import _native

MAX_RANKS = 8
PLAIN, ALLGATHER, REDUCE_SCATTER = 0, 1, 2
BF16, FP8_E4M3, FP16, FP32 = 0, 1, 2, 3

_VP = ctypes.c_void_p


class DenseArgs(ctypes.Structure):
    _fields_ = [
        ("a", _VP), ("b", _VP), ("d", _VP), ("bias", _VP),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldd", ctypes.c_int64),
        ("bias_row_stride", ctypes.c_int64),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32),
        ("mode", ctypes.c_int32), ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("group_m", ctypes.c_int32), ("num_sms", ctypes.c_int32), ("tile_n", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64),
        ("status", _VP),
        ("ag_land", _VP * MAX_RANKS), ("ag_flags", _VP * MAX_RANKS),
        ("start_ctr", _VP * MAX_RANKS),
        ("rs_stage", _VP * MAX_RANKS), ("rs_ctr", _VP * MAX_RANKS),
        ("rs_out", _VP), ("rs_work", _VP),
        ("stream", _VP),
    ]


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float8_e4m3fn:
        return FP8_E4M3
    if dt == torch.float16:
        return FP16
    if dt == torch.float32:
        return FP32
    raise TypeError(f"unsupported dtype {dt}")


def current_stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def fill_ptrs(arr, ptrs: Optional[Sequence[int]]) -> None:
    if ptrs is None:
        return
    for i, v in enumerate(ptrs):
        arr[i] = v


def run(args: DenseArgs) -> None:
    rc = _native.lib().fluxb_dense_gemm(ctypes.byref(args))
    _native.check(rc, "fluxb_dense_gemm")


def plain_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
               bias: Optional[torch.Tensor] = None, *, tile_n: int = 0, group_m: int = 0,
               num_sms: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = a[M,K] @ b[N,K]^T (+bias) on the tcgen05 kernel."""
    assert a.is_cuda and b.is_cuda and out.is_cuda, "the sm_100a GEMM needs CUDA tensors"
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == torch.bfloat16
    M, K = a.shape
    N = b.shape[0]
    args = DenseArgs()
    args.a, args.b, args.d = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.lda, args.ldb, args.ldd = a.stride(0), b.stride(0), out.stride(0)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.shape[-1] == N
        args.bias = bias.data_ptr()
        args.bias_row_stride = 0 if (bias.dim() == 1 or bias.shape[0] == 1) else bias.stride(0)
    args.M, args.N, args.K = M, N, K
    args.in_dtype = dtype_code(a.dtype)
    args.mode, args.rank, args.world = PLAIN, 0, 1
    args.group_m, args.num_sms, args.tile_n = group_m, num_sms, tile_n
    args.epoch = 1
    args.status = status.data_ptr() if status is not None else None
    args.stream = current_stream_ptr(a.device)
    run(args)
    return out
