"""Speed-of-light model for B200 (reference: ``python/flux/testing/gpu_perf_model.py``, which
tabulates A100/H100-class parts). Peaks come from ``MEASURED_PEAKS.json`` at the repository root
when present (copy bandwidth and cuBLAS bf16 throughput measured on this pool), otherwise from
the fallback figures 6650 GB/s and 1590 TFLOP/s; NVLink uses the measured 770 GB/s per direction."""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_NOMINAL_TFLOPS = {torch.bfloat16: 2250.0, torch.float16: 2250.0, torch.float8_e4m3fn: 4500.0,
                   torch.float8_e5m2: 4500.0, torch.float32: 1100.0}


def _peaks():
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"bf16": p["bf16_tflops"], "bf16_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "hbm": p["hbm_gbs"], "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


def get_tflops(dtype: torch.dtype = torch.bfloat16, sustained: bool = False) -> float:
    p = _peaks()
    base = p["bf16_sustained"] if sustained else p["bf16"]
    return base * _NOMINAL_TFLOPS.get(dtype, 2250.0) / 2250.0


def get_dram_gbps(device=None) -> float:
    return _peaks()["hbm"]


def get_nvlink_gbps() -> float:
    return 770.0


def estimate_gemm_sol_time_ms(M: int, N: int, K: int, dtype: torch.dtype = torch.bfloat16) -> float:
    elt = 1 if dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else 2
    t_flops = 2.0 * M * N * K / (get_tflops(dtype) * 1e9)
    t_mem = (M * K * elt + N * K * elt + M * N * 2) / (get_dram_gbps() * 1e6)
    return max(t_flops, t_mem)


def estimate_fused_sol_time_ms(flops_per_gpu: float, nvlink_bytes_per_gpu: float,
                               dtype: torch.dtype = torch.bfloat16, sustained: bool = False) -> float:
    """Roofline of a fused compute + collective kernel: the slower of the math at the measured
    GEMM peak and the bytes that must cross NVLink at the measured link bandwidth."""
    return max(flops_per_gpu / (get_tflops(dtype, sustained) * 1e9), nvlink_bytes_per_gpu / (get_nvlink_gbps() * 1e6))


def roofline_fraction(measured_ms: float, flops_per_gpu: float, nvlink_bytes_per_gpu: float = 0.0,
                      dtype: torch.dtype = torch.bfloat16, sustained: bool = False) -> float:
    return estimate_fused_sol_time_ms(flops_per_gpu, nvlink_bytes_per_gpu, dtype, sustained) / measured_ms
