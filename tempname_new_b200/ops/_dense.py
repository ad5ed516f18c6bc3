"""ctypes view of ``fluxb_dense_gemm`` (csrc/include/fluxb.h) shared by GemmOnly, AGKernel and
GemmRS."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from .. import _native

MAX_RANKS = 8
PLAIN, ALLGATHER, REDUCE_SCATTER = 0, 1, 2
ACT = {None: 0, "none": 0, "gelu": 1, "gelu_tanh": 1, "relu": 2, "silu": 3}
BF16, FP8_E4M3, FP16, FP32, FP8_E5M2, INT8 = 0, 1, 2, 3, 4, 5

_VP = ctypes.c_void_p


class DenseArgs(ctypes.Structure):
    _fields_ = [
        ("a", _VP), ("b", _VP), ("d", _VP), ("bias", _VP),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldd", ctypes.c_int64),
        ("bias_row_stride", ctypes.c_int64),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("scale_a", _VP), ("scale_b", _VP),
        ("mode", ctypes.c_int32), ("rank", ctypes.c_int32), ("world", ctypes.c_int32),
        ("group_m", ctypes.c_int32), ("num_sms", ctypes.c_int32), ("tile_n", ctypes.c_int32),
        ("act", ctypes.c_int32), ("cta_group", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("scale_flags", ctypes.c_uint32),
        ("timeout_ns", ctypes.c_uint64),
        ("status", _VP),
        ("ag_land", _VP * MAX_RANKS), ("ag_flags", _VP * MAX_RANKS),
        ("start_ctr", _VP * MAX_RANKS),
        ("rs_stage", _VP * MAX_RANKS), ("rs_ctr", _VP * MAX_RANKS),
        ("rs_out", _VP), ("wave_ctr", _VP), ("local_cnt", _VP),
        ("sa", _VP), ("sb", _VP), ("ag_scale_land", _VP * MAX_RANKS),
        ("blockscale", ctypes.c_int32), ("tile_m", ctypes.c_int32),
        ("stream", _VP),
        ("trace", _VP),
        ("b_kn", ctypes.c_int32), ("reserved_tail", ctypes.c_int32),
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
    if dt == torch.float8_e5m2:
        return FP8_E5M2
    if dt == torch.int8:
        return INT8
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


def check_scale(t: Optional[torch.Tensor], n_vec: int, what: str) -> bool:
    """A dequantisation scale is one number (per tensor) or one number per row of the input /
    per output column (the reference's int8 convention: input_scale [M, 1], weight_scale [1, N],
    python/flux/cpp_mod.pyi:352-353). Returns True for the vector form; anything else is refused
    rather than silently reduced to its first element."""
    if t is None or t.numel() == 1:
        return False
    if t.numel() == n_vec and max(t.shape) == n_vec:
        return True
    raise ValueError(f"{what} must hold 1 or {n_vec} values, got shape {tuple(t.shape)}")


def _as_scale(t: Optional[torch.Tensor], dev) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.float32 or t.device != dev:
        t = t.to(device=dev, dtype=torch.float32)
    return t.reshape(-1).contiguous()


_TIMELINE: Optional[torch.Tensor] = None

TRACE_SLOTS = ("entry", "handshake", "push_done", "first_tile_loads", "last_tile_loads", "first_store",
               "epilogue_done", "flag_wait_total") + tuple(f"slice{j}_ready" for j in range(8))


class KernelTimeline:
    """While active, every dense-kernel launch of this process writes a per-CTA timeline
    (``%globaltimer`` stamps) that ``summary()`` reduces to microseconds since the first CTA started:
    when the start handshake completed, when the pushes of the communication warps were published,
    when the loads of the first / last tile were issued, when the epilogue stored first / finished,
    and how long the producers waited for arrival flags in total. Only the latest launch is kept.
    ``slice{j}_ready``: post-attention mode - K slice j of the CTA's first tile became readable;
    reduce-scatter - ``slice0`` the first own tile was reached (two ranks), ``slice1`` / ``slice2`` the
    tail that sums the staging slabs was entered / left (three ranks and more).
    The reference exposes per-op ``profiling()`` context hooks (python/flux/cpp_mod.pyi); this is the
    device-side counterpart for the fused kernels here."""

    def __init__(self, device=None, ctas: int = 160):
        self.buf = torch.zeros(ctas, 16, dtype=torch.int64, device=device if device is not None else "cuda")

    def __enter__(self):
        global _TIMELINE
        _TIMELINE = self.buf
        return self

    def __exit__(self, *exc):
        global _TIMELINE
        _TIMELINE = None
        return False

    def summary(self) -> dict:
        t = self.buf.cpu()
        t = t[t[:, 0] > 0]
        if t.numel() == 0:
            return {}
        t0 = int(t[:, 0].min())
        out = {}
        for i, name in enumerate(TRACE_SLOTS):
            col = t[:, i]
            if i == 7:
                out[name + "_us"] = {"median": float(col.median()) / 1e3, "max": float(col.max()) / 1e3}
                continue
            col = col[col > 0]
            if col.numel():
                out[name + "_us"] = {"min": (int(col.min()) - t0) / 1e3, "median": (int(col.median()) - t0) / 1e3,
                                     "max": (int(col.max()) - t0) / 1e3}
        return out


def kn_in_place(w_nk: torch.Tensor) -> bool:
    """True when ``w_nk`` ([N, K] as the kernels see it) is a transposed view of [K, N] memory that the
    16-bit kernels can read without a copy (MN-major operand tiles): N contiguous, 16-byte aligned rows."""
    return (w_nk.dim() == 2 and w_nk.dtype in (torch.bfloat16, torch.float16) and w_nk.stride(0) == 1
            and w_nk.shape[0] % 8 == 0 and w_nk.stride(1) % 8 == 0 and w_nk.data_ptr() % 16 == 0
            and os.environ.get("FLUXB_KN_IN_PLACE", "1") != "0")


def base_args(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None, *,
              tile_n: int = 0, group_m: int = 0, num_sms: int = 0, act: Optional[str] = None,
              cta_group: int = 0, m: Optional[int] = None, tile_m: int = 0,
              status: Optional[torch.Tensor] = None, keep: Optional[list] = None) -> DenseArgs:
    """Fill the operand part of a DenseArgs for A[rows,K], B[N,K]. ``m`` is the number of output
    rows this GPU computes; when no tile knobs are given they come from the tuning table."""
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("the sm_100a GEMM kernels need CUDA tensors")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"shape mismatch: A {tuple(a.shape)} B {tuple(b.shape)} (B is [N, K])")
    # B is [N, K]; a transposed view of [K, N] memory (N contiguous) is read in place by the 16-bit kernels
    b_kn = b.stride(1) != 1 and kn_in_place(b)
    if b.stride(1) != 1 and not b_kn:
        b = b.contiguous()
        if keep is not None:
            keep.append(b)
    if a.stride(1) != 1:
        raise ValueError("A must have a contiguous K dimension")
    if a.dtype != b.dtype:
        raise TypeError("A and B must share a dtype")
    args = DenseArgs()
    if _TIMELINE is not None:
        _TIMELINE.zero_()
        args.trace = _TIMELINE.data_ptr()
    args.a, args.b = a.data_ptr(), b.data_ptr()
    args.lda, args.ldb = a.stride(0), (b.stride(1) if b_kn else b.stride(0))
    args.b_kn = 1 if b_kn else 0
    args._b_ref = b   # (a re-laid-out copy must outlive the launch)
    args.N, args.K = b.shape[0], a.shape[1]
    args.in_dtype = dtype_code(a.dtype)
    args.out_dtype = dtype_code(out_dtype)
    if bias is not None:
        if bias.dtype != out_dtype or bias.shape[-1] != b.shape[0] or bias.stride(-1) != 1:
            raise ValueError("bias must be [1|M, N] in the output dtype")
        args.bias = bias.data_ptr()
        args.bias_row_stride = 0 if (bias.dim() == 1 or bias.shape[0] == 1) else bias.stride(0)
    # per-row scales cover the rows of the whole problem (m), per-column scales the N outputs
    sa_vec = check_scale(scale_a, m if m is not None else a.shape[0], "input_scale")
    sb_vec = check_scale(scale_b, b.shape[0], "weight_scale")
    sa, sb = _as_scale(scale_a, a.device), _as_scale(scale_b, a.device)
    if sa is not None:
        args.scale_a = sa.data_ptr()
    if sb is not None:
        args.scale_b = sb.data_ptr()
    args.scale_flags = (1 if sa_vec else 0) | (2 if sb_vec else 0)
    if keep is not None:
        keep.extend([sa, sb])
    if tile_n == 0 and cta_group == 0 and m is not None:
        from ..tuning.table import lookup
        knobs = lookup(m, b.shape[0], a.shape[1], a.element_size())
        tile_n, cta_group = knobs["tile_n"], knobs["cta_group"]
        if group_m == 0:
            group_m = knobs["group_m"]
        if tile_m == 0:
            tile_m = knobs.get("tile_m", 0)
    args.group_m, args.num_sms, args.tile_n = group_m, num_sms, tile_n
    args.tile_m = tile_m
    args.act = ACT[act]
    args.cta_group = cta_group
    args.status = status.data_ptr() if status is not None else None
    args.stream = current_stream_ptr(a.device)
    return args


def plain_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
               bias: Optional[torch.Tensor] = None, scale_a: Optional[torch.Tensor] = None,
               scale_b: Optional[torch.Tensor] = None, *, tile_n: int = 0, group_m: int = 0,
               num_sms: int = 0, act: Optional[str] = None, cta_group: int = 0, tile_m: int = 0,
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = a[M,K] @ b[N,K]^T (* scales) (+bias) on the tcgen05 kernel."""
    keep: list = []
    args = base_args(a, b, bias, out.dtype, scale_a, scale_b, tile_n=tile_n, group_m=group_m,
                     num_sms=num_sms, act=act, cta_group=cta_group, m=a.shape[0], tile_m=tile_m,
                     status=status, keep=keep)
    if out.stride(1) != 1 or out.shape != (a.shape[0], b.shape[0]):
        raise ValueError("output must be [M, N] with contiguous rows")
    args.d, args.ldd = out.data_ptr(), out.stride(0)
    args.M = a.shape[0]
    args.mode, args.rank, args.world = PLAIN, 0, 1
    args.epoch = 1
    run(args)
    return out
