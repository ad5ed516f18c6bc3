"""Small utility ops: in-place fp32->bf16 cast, bitwise compare, uniform fill, MoE routing
indices (reference: ``flux.InplaceCast`` / ``inplace_cast_fp32_to_bf16``, ``flux.bitwise_check``,
``flux.uniform_initialize``, ``flux.calc_scatter_index``; ``src/pybind/inplace_cast.cc``,
``src/pybind/ths_op.cc:206-208,316-320``)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _native
from ..parallel.symm import FluxTimeoutError
from ._dense import current_stream_ptr, dtype_code

_CHUNK = 8192


class InplaceCast:
    """Casts an fp32 buffer to bf16 in place: afterwards ``t.view(torch.bfloat16)[:n]`` holds the
    result. ``data_size`` is the largest element count the object will be used with."""

    def __init__(self, data_size: int, device=None):
        self.data_size = int(data_size)
        self.epoch = 0
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        if self.device.type == "cuda":
            nflags = -(-self.data_size // _CHUNK) + 1
            self._scratch = torch.zeros(nflags + 1, dtype=torch.int32, device=self.device)
            self._status = torch.zeros(4, dtype=torch.int32, device=self.device)

    def from_fp32_to_bf16(self, t: torch.Tensor) -> torch.Tensor:
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("expected a contiguous float32 tensor")
        n = t.numel()
        if n > self.data_size:
            raise ValueError(f"InplaceCast was built for {self.data_size} elements, got {n}")
        if not t.is_cuda:
            src = t.reshape(-1).clone()
            t.view(torch.bfloat16).reshape(-1)[:n].copy_(src.to(torch.bfloat16))
            return t
        self.epoch += 1
        rc = _native.lib().fluxb_inplace_cast_fp32_to_bf16(
            ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(n),
            ctypes.c_void_p(self._scratch.data_ptr() + 4), ctypes.c_void_p(self._scratch.data_ptr()),
            ctypes.c_uint32(self.epoch), ctypes.c_uint64(2_000_000_000),
            ctypes.c_void_p(self._status.data_ptr()), ctypes.c_void_p(current_stream_ptr(t.device)))
        _native.check(rc, "fluxb_inplace_cast_fp32_to_bf16")
        return t

    def check_status(self) -> None:
        if self.device.type == "cuda" and self._status.tolist()[0] != 0:
            self._status.zero_()
            raise FluxTimeoutError("in-place cast: a chunk wait timed out")


def inplace_cast_fp32_to_bf16(t: torch.Tensor) -> torch.Tensor:
    return InplaceCast(t.numel(), t.device).from_fp32_to_bf16(t)


def bitwise_check(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True iff the two tensors hold the same bytes (shapes and dtypes must match)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    a, b = a.contiguous(), b.contiguous()
    if not a.is_cuda:
        return bool(torch.equal(a.view(torch.uint8), b.view(torch.uint8)))
    cnt = torch.zeros(1, dtype=torch.int64, device=a.device)
    rc = _native.lib().fluxb_bitwise_check(
        ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
        ctypes.c_int64(a.numel() * a.element_size()), ctypes.c_void_p(cnt.data_ptr()),
        ctypes.c_void_p(current_stream_ptr(a.device)))
    _native.check(rc, "fluxb_bitwise_check")
    return int(cnt.item()) == 0


def uniform_initialize(t: torch.Tensor, seed: int, min_val: float, max_val: float) -> torch.Tensor:
    """Fill ``t`` with uniform values in [min_val, max_val) from a counter-based generator
    (the same seed gives the same tensor on every rank)."""
    if not t.is_cuda:
        g = torch.Generator().manual_seed(int(seed))
        t.copy_((torch.rand(t.shape, generator=g) * (max_val - min_val) + min_val).to(t.dtype))
        return t
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    rc = _native.lib().fluxb_uniform_fill(
        ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(t.numel()), dtype_code(t.dtype),
        ctypes.c_uint64(int(seed)), ctypes.c_float(min_val), ctypes.c_float(max_val),
        ctypes.c_void_p(current_stream_ptr(t.device)))
    _native.check(rc, "fluxb_uniform_fill")
    return t


def moe_index_build(choosed_experts: torch.Tensor, num_experts: int, topk: Optional[int] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable routing indices from ``choosed_experts [tokens, topk]`` (or flat): returns
    ``(splits [E], offsets [E+1], scatter_index (same shape), gather_index [n], topk_index [n])``
    — all on the device, without a host synchronisation."""
    ce = choosed_experts
    if topk is None:
        topk = ce.shape[1] if ce.dim() == 2 else 1
    flat = ce.reshape(-1).to(torch.int32).contiguous()
    n = flat.numel()
    if not flat.is_cuda:
        order = torch.argsort(flat, stable=True)
        scatter = torch.empty_like(flat)
        scatter[order] = torch.arange(n, dtype=torch.int32)
        splits = torch.bincount(flat.long(), minlength=num_experts).to(torch.int32)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int32), splits.cumsum(0).to(torch.int32)])
        return splits, offsets, scatter.view(ce.shape), (order // topk).to(torch.int32), (order % topk).to(torch.int32)
    dev = flat.device
    lib = _native.lib()
    lib.fluxb_moe_index_scratch_elems.restype = ctypes.c_int64
    scratch = torch.empty(int(lib.fluxb_moe_index_scratch_elems(ctypes.c_int64(n), num_experts)),
                          dtype=torch.int32, device=dev)
    splits = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    scatter = torch.empty(n, dtype=torch.int32, device=dev)
    gather = torch.empty(n, dtype=torch.int32, device=dev)
    tki = torch.empty(n, dtype=torch.int32, device=dev)
    rc = lib.fluxb_moe_index_build(
        ctypes.c_void_p(flat.data_ptr()), ctypes.c_int64(n), num_experts, topk,
        ctypes.c_void_p(splits.data_ptr()), ctypes.c_void_p(offsets.data_ptr()),
        ctypes.c_void_p(scatter.data_ptr()), ctypes.c_void_p(gather.data_ptr()),
        ctypes.c_void_p(tki.data_ptr()), ctypes.c_void_p(scratch.data_ptr()),
        ctypes.c_void_p(current_stream_ptr(dev)))
    _native.check(rc, "fluxb_moe_index_build")
    return splits, offsets, scatter.view(ce.shape), gather, tki


def calc_scatter_index(choosed_experts: torch.Tensor, splits: torch.Tensor) -> torch.Tensor:
    """Destination row of every (token, k) entry in expert-sorted order (reference:
    ``flux.calc_scatter_index(choosed_experts, splits)``; unlike the reference kernel the result
    is stable, i.e. equal to ``argsort(argsort(experts, stable))``)."""
    return moe_index_build(choosed_experts, splits.numel())[2]
