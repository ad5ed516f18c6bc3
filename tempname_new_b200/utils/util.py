"""Small helpers with the names of the reference's ``flux.util`` (``python/flux/util.py:31-214``):
architecture query, tolerance check with a readable report, profiler contexts that merge the
per-rank chrome traces, CUDA-event timing."""
from __future__ import annotations

import contextlib
import gzip
import json
import os
import pathlib
import shutil
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def get_arch() -> int:
    """Compute capability of the current device as major*10+minor (100 on B200)."""
    if not torch.cuda.is_available():
        return 0
    major, minor = torch.cuda.get_device_capability()
    return major * 10 + minor


def is_fp8_dtype(dtype: torch.dtype) -> bool:
    return dtype in (torch.float8_e4m3fn, torch.float8_e5m2)


def torch_allclose(x: torch.Tensor, y: torch.Tensor, rtol: float, atol: float, verbose: bool = True) -> None:
    """Raise with the worst offenders listed if ``|x - y| <= atol + rtol * |y|`` fails anywhere."""
    xf, yf = x.float(), y.float()
    bad = ~torch.isclose(xf, yf, rtol=rtol, atol=atol)
    if not bad.any():
        return
    n = int(bad.sum())
    msg = [f"{n} of {x.numel()} elements differ (rtol={rtol}, atol={atol})"]
    if verbose:
        diff = (xf - yf).abs()
        flat = torch.where(bad, diff, torch.zeros_like(diff)).reshape(-1)
        for i in torch.topk(flat, min(5, n)).indices.tolist():
            idx = tuple(int(v) for v in torch.unravel_index(torch.tensor(i), x.shape))
            msg.append(f"  at {idx}: {xf.reshape(-1)[i].item():.6g} vs {yf.reshape(-1)[i].item():.6g}")
    raise AssertionError("\n".join(msg))


@contextlib.contextmanager
def with_torch_deterministic(mode: bool, warn_only: bool = True):
    old, old_warn = torch.are_deterministic_algorithms_enabled(), torch.is_deterministic_algorithms_warn_only_enabled()
    torch.use_deterministic_algorithms(mode, warn_only=warn_only)
    try:
        yield
    finally:
        torch.use_deterministic_algorithms(old, warn_only=old_warn)


def get_torch_prof_ctx(do_prof: bool):
    if not do_prof:
        return contextlib.nullcontext()
    return torch.profiler.profile(
        activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
        record_shapes=True, with_stack=False)


def _merge_traces(files: List[pathlib.Path], out: pathlib.Path) -> None:
    """One chrome trace with every rank's events; pids are offset per rank so they do not clash."""
    events = []
    for rank, f in enumerate(files):
        opener = gzip.open if f.suffix == ".gz" else open
        with opener(f, "rt") as fh:
            data = json.load(fh)
        for ev in data.get("traceEvents", []):
            for key in ("pid", "tid"):
                if isinstance(ev.get(key), int):
                    ev[key] = ev[key] + rank * 1_000_000
            if ev.get("ph") == "M" and ev.get("name") == "process_name":
                ev.setdefault("args", {})["name"] = f"rank{rank} " + str(ev["args"].get("name", ""))
            events.append(ev)
    with gzip.open(out, "wt") as fh:
        json.dump({"traceEvents": events}, fh)


class group_profile:
    """``with group_profile("name", do_prof, group=pg): ...`` profiles every rank and leaves
    ``prof/<name>/trace_merged.json.gz`` on rank 0."""

    def __init__(self, name: Optional[str] = None, do_prof: bool = True, merge_group=None, keep_merged_only: bool = True,
                 group=None):
        self.name = name or "fluxb"
        self.do_prof = do_prof
        self.group = group if group is not None else merge_group
        self.keep_merged_only = keep_merged_only
        self.prof = None

    def __enter__(self):
        if self.do_prof:
            self.prof = get_torch_prof_ctx(True)
            self.prof.__enter__()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        if not self.do_prof:
            return False
        self.prof.__exit__(exc_type, exc_val, exc_tb)
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        outdir = pathlib.Path("prof") / self.name
        outdir.mkdir(parents=True, exist_ok=True)
        mine = outdir / f"rank{rank}.json"
        self.prof.export_chrome_trace(str(mine))
        if dist.is_initialized() and world > 1:
            dist.barrier(group=self.group)
        if rank == 0:
            files = [outdir / f"rank{r}.json" for r in range(world)]
            _merge_traces([f for f in files if f.exists()], outdir / "trace_merged.json.gz")
            if self.keep_merged_only:
                for f in files:
                    with contextlib.suppress(OSError):
                        f.unlink()
        return False


def bench_func(func: Callable, iters: int, warmup_iters: int):
    """(last result, milliseconds per call) measured with CUDA events on the current stream."""
    out = None
    for _ in range(warmup_iters):
        out = func()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        out = func()
    stop.record()
    stop.synchronize()
    return out, start.elapsed_time(stop) / max(iters, 1)
