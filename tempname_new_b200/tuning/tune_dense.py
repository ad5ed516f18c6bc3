"""Sweep the dense kernel's knobs for one or more shapes on the current GPU and print the
winners as ``DENSE_TABLE`` entries (the role of the reference's ``tools/tune_gemm_only.py``).

    python -m tempname_new_b200.tuning.tune_dense --shape 8192,6144,12288 --shape 8192,12288,6144

Every candidate runs back to back for ``--seconds`` (default 0.5 s): on a 1 kW part the power cap,
not the boost clock of an isolated launch, decides which tile shape wins.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import _dense
from .table import candidates


def sustained_ms(fn, seconds: float) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    iters = max(5, int(seconds * 1e3 / max(s.elapsed_time(e), 1e-3)))
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def tune(m: int, n: int, k: int, seconds: float = 0.5, verbose: bool = False, dtype=torch.bfloat16):
    dev = torch.device("cuda")
    a = torch.randn(m, k, device=dev).to(dtype)
    b = (torch.randn(n, k, device=dev) * 0.02).to(dtype)
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    t_ref = sustained_ms(lambda: torch.matmul(a, b.t(), out=out), seconds) if dtype == torch.bfloat16 else None
    res = []
    for knobs in candidates(m, n, k):
        ms = sustained_ms(lambda: _dense.plain_gemm(a, b, out, **knobs), seconds)
        res.append((ms, knobs))
        if verbose:
            print(f"  {knobs}: {ms:.3f} ms", flush=True)
    res.sort(key=lambda r: r[0])
    ms, best = res[0]
    tf = 2.0 * m * n * k / 1e9
    return {"key": [m, n, k], "best": best, "ms": ms, "tflops": tf / ms, "cublas_ms": t_ref,
            "cublas_tflops": tf / t_ref if t_ref else None,
            "runner_up": [dict(r[1], ms=r[0]) for r in res[1:4]]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", required=True, help="M,N,K")
    ap.add_argument("--seconds", type=float, default=0.5)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float8_e4m3fn
    for s in args.shape:
        m, n, k = (int(v) for v in s.split(","))
        print(json.dumps(tune(m, n, k, args.seconds, args.verbose, dt)), flush=True)


if __name__ == "__main__":
    main()
