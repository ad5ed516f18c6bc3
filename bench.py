#!/usr/bin/env python
"""Headline benchmark: the tensor-parallel MLP block of GPT-3-175B (hidden 12288, ffn 49152,
8192 tokens) as AG+GEMM followed by GEMM+RS, bf16, TP = number of GPUs.

    python bench.py --gpus N --steps K --warmup W            # this library (default)
    python bench.py --impl reference ...                     # the reference (unavailable here)
    python bench.py --impl torch ...                         # torch.matmul + NCCL as the headline arm

The default arm also times the torch.matmul + NCCL block in the same process (half of its steps
before and half after the headline steps) and prints ``vs_baseline`` = headline / that baseline, checks
the two arms against each other before timing (``verified``), and adds a >= 2 s sustained loop.

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...``. Rank 0 prints one JSON line.

A step is: all-gather the sequence-sharded activations [8192/N, 12288] fused into the fc1 GEMM
(weight shard [49152/N, 12288]), then the fc2 GEMM (weight shard [12288, 49152/N]) fused with
the reduce-scatter back to [8192/N, 12288]. Total work is fixed as N grows (strong scaling):
4 * 8192 * 12288 * 49152 FLOP per step over the whole job.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOKENS, HIDDEN, FFN = 8192, 12288, 49152
METRIC = "fused-op TFLOPS (AG-GEMM + GEMM-RS, GPT-3-175B TP MLP shapes)"
REFERENCE_UNAVAILABLE = (
    "reference (Flux 1.1.2 fork) cannot be installed offline: pip install --no-index of the reference tree "
    "fails (setup.py tries to download a cached wheel, then builds with no sources because 3rdparty/cutlass, "
    "3rdparty/nccl are empty submodules and NVSHMEM is absent); it also has no sm_100 kernels")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fluxb", choices=["fluxb", "reference", "torch"])
    ap.add_argument("--tokens", type=int, default=TOKENS)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the benchmark runs (read-only). Every
    timed region is marked with a label; ``summary(label)`` reduces the samples taken inside the
    regions of that label."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.windows = []
        self.rows = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self, label, t0, t1):
        self.windows.append((label, t0, t1))

    def stop(self):
        if self.proc is None:
            self.rows = []
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        rows = []
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), float(parts[4]), parts[5:9]))
            except ValueError:
                continue
        self.rows = rows

    def summary(self, label):
        rows = self.rows or []
        wins = [(a, b) for (l, a, b) in self.windows if l == label]
        sel = [r for r in rows if any(a - 0.03 <= r[0] <= b + 0.03 for a, b in wins)]
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": rows[0][2] if rows else None, "reasons": [], "samples": 0}
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in sel:
            for n, v in zip(names, r[4]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {
            "sm_mhz": statistics.median(r[1] for r in sel),
            "sm_max_mhz": sel[0][2],
            "power_w": statistics.median(r[3] for r in sel),
            "reasons": sorted(reasons),
            "samples": len(sel),
        }


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pg = dist.group.WORLD

    import tempname_new_b200 as flux
    from tempname_new_b200 import _native
    from tempname_new_b200.models.tp_mlp import TPMLP, HostStep

    flux.init_flux_shm(pg)
    M = args.tokens
    seg = M // world
    torch.manual_seed(1234 + rank)
    x = torch.randn(seg, HIDDEN, device=dev).bfloat16()          # inputs N(0,1)
    x_pinned = torch.randn(seg, HIDDEN).bfloat16().pin_memory()
    flops_step = 4.0 * M * HIDDEN * FFN
    res_pinned = torch.empty(1 + HIDDEN, dtype=torch.float32).pin_memory()

    # one set of weights N(0, 0.02) for both arms
    mlp = TPMLP(HIDDEN, FFN, pg, bias=False, dtype=torch.bfloat16, device=dev, act="none")
    mlp.requires_grad_(False)
    w1, w2 = mlp.fc1.weight.detach(), mlp.fc2.weight.detach()

    @torch.no_grad()
    def fluxb_step(xin=None):
        return mlp(x if xin is None else xin)

    # the operative baseline: the same block on torch.matmul (cuBLAS) + NCCL, the composition the
    # reference's own tests time as "torch" (test/python/gemm_rs/test_gemm_rs.py:57-156)
    full = torch.empty(M, HIDDEN, device=dev, dtype=torch.bfloat16) if world > 1 else None
    out_t = torch.empty(seg, HIDDEN, device=dev, dtype=torch.bfloat16)

    @torch.no_grad()
    def torch_step(xin=None):
        xin = x if xin is None else xin
        if world > 1:
            dist.all_gather_into_tensor(full, xin)
            h = torch.matmul(full, w1.t())
            part = torch.matmul(h, w2.t())
            dist.reduce_scatter_tensor(out_t, part)
            return out_t
        h = torch.matmul(xin, w1.t())
        return torch.matmul(h, w2.t(), out=out_t)

    fluxb_e2e_step = HostStep(fluxb_step, dev)
    torch_e2e_step = HostStep(torch_step, dev)

    def fluxb_e2e():
        return fluxb_e2e_step(x_pinned, res_pinned)

    def torch_e2e():
        return torch_e2e_step(x_pinned, res_pinned)

    # ---- the two arms must agree before anything is timed
    y_f = fluxb_step().float()
    y_t = torch_step().float()
    torch.cuda.synchronize()
    err = (y_f - y_t).abs().max()
    scale = y_t.abs().max().clamp_min(1e-6)
    v = torch.stack([err, scale]).double()
    dist.all_reduce(v, op=dist.ReduceOp.MAX)
    max_err, ref_max = float(v[0]), float(v[1])
    mlp.fc1._cache.ag(M, FFN // world, HIDDEN, torch.bfloat16).check_status()
    mlp.fc2._cache.rs(M, HIDDEN, torch.bfloat16).check_status()
    verified = bool(max_err <= 2e-2 * max(1.0, ref_max))
    del y_f, y_t

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    def timed(fn, steps, warmup, label):
        """(ms per step on the device, max over ranks; host us per step spent enqueueing)"""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        t_host = time.time()
        torch.cuda.synchronize()
        t1 = time.time()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if sampler:
            sampler.mark(label, t0, t1)
        return float(ms.item()) / steps, (t_host - t0) * 1e6 / steps

    warmup = max(args.warmup, 3)
    K = args.steps
    half = max((K + 1) // 2, 1)
    only_torch = args.impl == "torch"

    def tf(ms):
        return flops_step / ms / 1e9

    # ---- device-timed: baseline half, the K headline steps, baseline half (same thermal state on
    # both sides of the headline)
    bt_a, _ = timed(torch_step, half, warmup, "torch")
    launches0 = _native.launch_count()
    if only_torch:
        ms_step, host_us = timed(torch_step, K, warmup, "headline")
    else:
        ms_step, host_us = timed(fluxb_step, K, warmup, "headline")
    launches = _native.launch_count() - launches0
    launches_timed = launches * K // (K + warmup)   # the warm-up steps launched the same kernels
    bt_b, _ = timed(torch_step, half, warmup, "torch")
    ms_base = 0.5 * (bt_a + bt_b)

    # ---- end to end through the public API: pinned host shard -> device, block, result -> host
    e2e = base_e2e = None
    if not args.no_e2e:
        be_a, _ = timed(torch_e2e, half, warmup, "torch_e2e")
        ms_e2e, host_us_e2e = timed(torch_e2e if only_torch else fluxb_e2e, K, warmup, "e2e")
        be_b, _ = timed(torch_e2e, half, warmup, "torch_e2e")
        ms_base_e2e = 0.5 * (be_a + be_b)
        e2e = {"value": tf(ms_e2e), "unit": "TFLOPS", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": x_pinned.numel() * x_pinned.element_size(),
               "d2h_bytes_per_step": res_pinned.numel() * res_pinned.element_size(),
               "host_us_per_step": host_us_e2e}
        base_e2e = {"value": tf(ms_base_e2e), "ms_per_step": ms_base_e2e}

    # ---- sustained: at least 2 s of back-to-back steps per arm, so that the power cap (not the
    # boost clock of a short burst) sets the SM clock
    sustained = None
    if not args.no_sustained:
        n_f = max(int(2000.0 / ms_step) + 1, K)
        n_t = max(int(2000.0 / ms_base) + 1, K)
        st_t_a, _ = timed(torch_step, (n_t + 1) // 2, 2, "torch_sustained")
        st_f, _ = timed(torch_step if only_torch else fluxb_step, n_f, 2, "sustained")
        st_t_b, _ = timed(torch_step, (n_t + 1) // 2, 2, "torch_sustained")
        sustained = {"steps": n_f, "ms_per_step": st_f, "value": tf(st_f),
                     "baseline_ms_per_step": 0.5 * (st_t_a + st_t_b), "baseline_value": tf(0.5 * (st_t_a + st_t_b))}
        sustained["ratio"] = sustained["value"] / sustained["baseline_value"]

    # informational: each fused op alone against its roofline
    extra = {}
    if not only_torch:
        op_ag = mlp.fc1._cache.ag(M, FFN // world, HIDDEN, torch.bfloat16)
        op_rs = mlp.fc2._cache.rs(M, HIDDEN, torch.bfloat16)
        h = torch.empty(M, FFN // world, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            extra["ag_gemm_ms"], _ = timed(lambda: op_ag.forward(x, mlp.fc1.weight, output=h), 10, 3, "ops")
            extra["gemm_rs_ms"], _ = timed(lambda: op_rs.forward(h, mlp.fc2.weight), 10, 3, "ops")
        op_ag.check_status()
        op_rs.check_status()
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
        link_gbs = 770.0
        half_flops = flops_step / 2 / world
        t_compute = half_flops / (peak_tf * 1e9)                           # ms per op per GPU
        ag_bytes = (world - 1) / world * M * HIDDEN * 2
        rs_bytes = (world - 1) / world * M * HIDDEN * 2
        extra["roofline"] = {
            "peak_tflops": peak_tf, "peak_source": "measured sustained" if peaks else "fallback",
            "nvlink_gbs": link_gbs,
            "ag_gemm_frac": max(t_compute, ag_bytes / (link_gbs * 1e6)) / extra["ag_gemm_ms"],
            "gemm_rs_frac": max(t_compute, rs_bytes / (link_gbs * 1e6)) / extra["gemm_rs_ms"],
        }

    if sampler:
        sampler.stop()

    if rank == 0:
        clocks = sampler.summary("headline")
        base_clocks = sampler.summary("torch")
        value = tf(ms_step)
        base_value = tf(ms_base)

        def per_mhz(val, clk):
            return val / world / clk["sm_mhz"] if clk.get("sm_mhz") else None

        if sustained is not None:
            sc, sbc = sampler.summary("sustained"), sampler.summary("torch_sustained")
            sustained.update(clocks=sc, baseline_clocks=sbc,
                             tflops_per_gpu_per_mhz=per_mhz(sustained["value"], sc),
                             baseline_tflops_per_gpu_per_mhz=per_mhz(sustained["baseline_value"], sbc))
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world,
            "steps": K, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong",
            # the reference publishes no B200 number; the baseline is torch.matmul + NCCL on the same
            # box, timed here in the same process around the headline steps
            "vs_baseline": value / base_value,
            "baseline": {"impl": "torch.matmul (cuBLAS) + NCCL all_gather_into_tensor / reduce_scatter_tensor",
                         "value": base_value, "ms_per_step": ms_base, "ratio": value / base_value,
                         "e2e": base_e2e,
                         "e2e_ratio": (e2e["value"] / base_e2e["value"]) if e2e else None,
                         "clocks": base_clocks, "steps": [half, half],
                         "order": "baseline half, headline, baseline half"},
            "verified": verified, "max_err": max_err, "ref_abs_max": ref_max,
            "dtype": "bf16", "data": "synthetic",
            "impl": "torch_nccl" if only_torch else "fluxb",
            "config": {"model": "GPT-3-175B TP MLP block (AG-GEMM M=8192 K=12288 N=49152/W; GEMM-RS M=8192 "
                                "K=49152/W N=12288)", "global_batch": M, "seq_len": M,
                       "parallelism": f"tp{world}",
                       "l2": "weights (>=151 MB per GEMM) exceed the 126 MB L2, no extra flush"},
            "clocks": clocks, "tflops_per_gpu_per_mhz": per_mhz(value, clocks),
            "e2e": e2e, "sustained": sustained,
            "host_us_per_step": host_us,
            "gpu_launches": max(launches_timed, 0),
        }
        line.update(extra)
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if verified else 1


if __name__ == "__main__":
    sys.exit(main())
