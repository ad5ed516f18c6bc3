"""Time the grouped (MoE) GEMM paths for one problem on the current GPU and print one JSON line per
path - the role of the reference's ``tools/tune_gemm_grouped_v3_only.py``. The grouped kernel has no
per-shape tile table (its column width follows N); what can be chosen is how gathered rows reach the
kernel, so that is what this sweeps: the sorted-buffer gather (default), the ``cp.async`` row gather
and the ``tile::gather4`` loader, selected through ``FLUXB_MOE_GATHER`` in child processes.

    python -m tempname_new_b200.tuning.tune_grouped --rows 65536 --n 3072 --k 4096 --experts 8
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    base = [sys.executable, "-m", "tempname_new_b200.utils.microbench", "grouped", "--rows", str(args.rows),
            "--n", str(args.n), "--k", str(args.k), "--experts", str(args.experts), "--topk", str(args.topk),
            "--iters", str(args.iters)]
    results = []
    for name, extra, env in (("contiguous", [], {}),
                             ("gathered, sorted buffer", ["--gathered"], {"FLUXB_MOE_GATHER": "pregather"}),
                             ("gathered, cp.async", ["--gathered"], {"FLUXB_MOE_GATHER": "cpasync"}),
                             ("gathered, tile::gather4", ["--gathered"], {"FLUXB_MOE_GATHER": "gather4"})):
        r = subprocess.run(base + extra, capture_output=True, text=True, env=dict(os.environ, **env))
        line = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if r.returncode != 0 or not line:
            results.append({"path": name, "error": (r.stderr or r.stdout)[-300:]})
            continue
        d = json.loads(line[-1])
        d["path"] = name
        results.append(d)
        print(json.dumps(d), flush=True)
    ok = [d for d in results if "ms" in d and d["path"].startswith("gathered")]
    if ok:
        best = min(ok, key=lambda d: d["ms"])
        print(json.dumps({"best_gather_path": best["path"], "ms": best["ms"]}))


if __name__ == "__main__":
    main()
