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


# ------------------------------------------------------------------------------------------
# Device queries and clock-based peaks (reference: python/flux/testing/gpu_perf_model.py:29-160,
# 198-262, written there for sm80/sm90 parts). On B200 a tcgen05 tensor core retires, per SM and
# clock, 8192 dense FLOP in bf16/fp16, twice that in fp8/int8 and half in tf32; the fp32 SIMD
# lanes 256. Without a GPU the functions fall back to the nominal part: 148 SMs, 1965 MHz, 227 KB.
# ------------------------------------------------------------------------------------------
_TC_FLOP_PER_SM_CLK = {torch.bfloat16: 8192, torch.float16: 8192, torch.int16: 8192, torch.float32: 4096,
                       torch.int32: 4096, torch.float8_e4m3fn: 16384, torch.float8_e5m2: 16384, torch.int8: 16384}
_SIMD_FLOP_PER_SM_CLK = {torch.float32: 256, torch.float16: 512, torch.bfloat16: 512}
_DRAM_GBPS_BY_NAME = {"NVIDIA B200": 7700.0, "NVIDIA H100 80GB HBM3": 3350.0, "NVIDIA H800": 3350.0,
                      "NVIDIA A100-SXM4-80GB": 2039.0, "NVIDIA A100 80GB PCIe": 1935.0}


def is_fp8_dtype(dtype: torch.dtype) -> bool:
    return dtype.itemsize == 1 and dtype.is_floating_point


def nvsmi(attrs):
    """``nvidia-smi --query-gpu`` of GPU 0, integer fields only."""
    import subprocess
    out = subprocess.check_output(["nvidia-smi", "-i", "0", "--query-gpu=" + ",".join(attrs),
                                   "--format=csv,noheader,nounits"])
    return [int(v) for v in out.decode().split(",")]


def get_clock_rate_in_khz() -> float:
    try:
        return nvsmi(["clocks.max.sm"])[0] * 1e3
    except Exception:
        return 1965e3


def get_device_property(device=None):
    return torch.cuda.get_device_properties(device)


def get_device_multi_processor_count(device=None) -> int:
    return get_device_property(device).multi_processor_count if torch.cuda.is_available() else 148


def get_device_shared_memory_size() -> int:
    """Shared memory per SM in bytes."""
    if torch.cuda.is_available():
        p = get_device_property(torch.cuda.current_device())
        return int(getattr(p, "shared_memory_per_multiprocessor", 233472))
    return 233472


def get_max_tensorcore_tflops(dtype: torch.dtype, clock_rate: float, device=None) -> float:
    """Dense tensor-core peak at ``clock_rate`` (kHz) over all SMs."""
    if dtype not in _TC_FLOP_PER_SM_CLK:
        raise RuntimeError(f"dtype {dtype} has no tensor-core rate")
    return get_device_multi_processor_count(device) * clock_rate * 1e3 * _TC_FLOP_PER_SM_CLK[dtype] * 1e-12


def get_max_simd_tflops(dtype: torch.dtype, clock_rate: float, device=None) -> float:
    if dtype not in _SIMD_FLOP_PER_SM_CLK:
        raise RuntimeError(f"dtype {dtype} has no SIMD rate")
    return get_device_multi_processor_count(device) * clock_rate * 1e3 * _SIMD_FLOP_PER_SM_CLK[dtype] * 1e-12


def _share(device, num_ctas: int) -> float:
    # one CTA per SM drives the SM's tensor core (tcgen05 is issued by one thread per CTA)
    sms = get_device_multi_processor_count(device)
    return min(sms, max(num_ctas, 0)) / sms


def get_tensorcore_tflops(device, num_ctas: int, num_warps: int, dtype: torch.dtype) -> float:
    return _share(device, num_ctas) * get_max_tensorcore_tflops(dtype, get_clock_rate_in_khz(), device)


def get_simd_tflops(device, num_ctas: int, num_warps: int, dtype: torch.dtype) -> float:
    sms = get_device_multi_processor_count(device)
    frac = min(sms * 4, num_ctas * min(num_warps, 4)) / (sms * 4)
    return frac * get_max_simd_tflops(dtype, get_clock_rate_in_khz(), device)


def get_tflops_approx(device, num_ctas: int, num_warps: int, dtype: torch.dtype) -> float:
    return get_tensorcore_tflops(device, num_ctas, num_warps, dtype)


def get_full_tflops_approx(dtype: torch.dtype, device=None) -> float:
    return get_tflops_approx(device, get_device_multi_processor_count(device), 4, dtype)


def get_dram_gbps_by_device_name(device_name: str) -> float:
    if device_name not in _DRAM_GBPS_BY_NAME:
        raise KeyError(f"no DRAM bandwidth on record for {device_name!r}")
    return _DRAM_GBPS_BY_NAME[device_name]


def _out_dtype(input_dtype: torch.dtype) -> torch.dtype:
    return torch.bfloat16 if input_dtype.itemsize == 1 else input_dtype


def print_gemm_sol_time(M: int, N: int, K: int, input_dtype: torch.dtype, output_dtype=None):
    """(tensor-core, read, write) milliseconds of a GEMM at the measured peaks; also printed."""
    output_dtype = output_dtype or _out_dtype(input_dtype)
    t_c = 2.0 * M * N * K / 1e9 / get_tflops(input_dtype)
    t_r = (M * K + N * K) * input_dtype.itemsize / 1e6 / get_dram_gbps()
    t_w = M * N * output_dtype.itemsize / 1e6 / get_dram_gbps()
    print(f"SOL gemm: tensor core {t_c:0.3f} ms, memory read {t_r:0.3f} ms, write {t_w:0.3f} ms")
    return t_c, t_r, t_w


def print_grouped_gemm_sol_time_ms(M: int, N: int, K: int, E: int, input_dtype: torch.dtype, output_dtype=None,
                                   num_groups: int = 1):
    output_dtype = output_dtype or _out_dtype(input_dtype)
    t_c = 2.0 * M * N * K * num_groups / 1e9 / get_tflops(input_dtype)
    t_r = (M * K + N * K * E) * input_dtype.itemsize * num_groups / 1e6 / get_dram_gbps()
    t_w = M * N * output_dtype.itemsize * num_groups / 1e6 / get_dram_gbps()
    print(f"SOL grouped gemm: tensor core {t_c:0.3f} ms, memory read {t_r:0.3f} ms, write {t_w:0.3f} ms")
    return t_c, t_r, t_w
