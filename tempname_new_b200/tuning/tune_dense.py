"""Sweep the dense kernel's knobs for one or more shapes on the current GPU and print the
winners as ``DENSE_TABLE`` entries (the role of the reference's ``tools/tune_gemm_only.py``).

    python -m tempname_new_b200.tuning.tune_dense --shape 8192,6144,12288 --shape 8192,12288,6144
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import _dense
from ..utils.microbench import timed

CANDIDATES = [(cg, bn, gm) for cg in (1, 2) for bn in (256, 192, 128) for gm in (2, 4, 8, 16)
              if not (cg == 2 and gm == 16)]


def tune(m: int, n: int, k: int, iters: int = 5, verbose: bool = False):
    dev = torch.device("cuda")
    a = torch.randn(m, k, device=dev).bfloat16()
    b = (torch.randn(n, k, device=dev) * 0.02).bfloat16()
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    t_ref = timed(lambda: torch.matmul(a, b.t(), out=out), iters, 2)
    res = []
    for cg, bn, gm in CANDIDATES:
        ms = timed(lambda: _dense.plain_gemm(a, b, out, tile_n=bn, group_m=gm, cta_group=cg), iters, 2)
        res.append((ms, cg, bn, gm))
        if verbose:
            print(f"  cg{cg} bn{bn} g{gm}: {ms:.3f} ms", flush=True)
    res.sort()
    ms, cg, bn, gm = res[0]
    tf = 2.0 * m * n * k / 1e9
    return {"key": [m, n, k], "best": {"cta_group": cg, "tile_n": bn, "group_m": gm}, "ms": ms,
            "tflops": tf / ms, "cublas_ms": t_ref, "cublas_tflops": tf / t_ref,
            "runner_up": [{"cta_group": r[1], "tile_n": r[2], "group_m": r[3], "ms": r[0]} for r in res[1:4]]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", required=True, help="M,N,K")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    for s in args.shape:
        m, n, k = (int(v) for v in s.split(","))
        print(json.dumps(tune(m, n, k, args.iters, args.verbose)), flush=True)


if __name__ == "__main__":
    main()
