"""``op.profiling(...)`` support (reference: ``ProfilingContext`` / ``TuningRecord`` in
``src/ths_op/ths_op.cc:105-320`` and the sweep drivers ``tools/tune_*.py``).

The reference iterates every registered CUTLASS hparams set and prints C++ registration code.
Here a kernel family has a handful of run-time knobs (tile_n, raster group, SM count), so a
profile run times each candidate with CUDA events (max over ranks) and records the winner in a
``ProfilingContext`` that can be dumped as a JSON tuning table."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass
class TuningRecord:
    op: str
    key: Dict
    best: Dict
    ms: float


@dataclass
class ProfilingContext:
    name: str = "fluxb"
    records: List[TuningRecord] = field(default_factory=list)
    results: List[str] = field(default_factory=list)

    def add(self, rec: TuningRecord) -> None:
        self.records.append(rec)
        self.results.append(f"{rec.op} {rec.key} -> {rec.best} {rec.ms:.4f} ms")

    def get_code(self) -> str:
        return json.dumps([asdict(r) for r in self.records], indent=1)

    def get_all_prof_results(self) -> List[str]:
        return list(self.results)

    def get_latest_prof_result(self) -> str:
        return self.results[-1] if self.results else ""

    def get_latest_record(self) -> Optional[TuningRecord]:
        return self.records[-1] if self.records else None

    def get_all_records(self) -> List[TuningRecord]:
        return list(self.records)


def time_cuda(fn: Callable[[], object], warmup: int = 5, iters: int = 10, group=None) -> float:
    """Median milliseconds per call, measured with CUDA events; max over the ranks of ``group``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    ms = times[len(times) // 2]
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        ms = float(t.item())
    return ms


def profile_call(op, name: str, fn: Callable[[], object], prof_ctx: Optional[ProfilingContext],
                 key=None, segmented_rows: int = 0):
    """Run ``fn`` (one call of a fused op). With a ``ProfilingContext`` on a GPU: time it - for the ops
    built on the dense kernel (``key`` = the (M, N, K) their knobs are looked up under) once per
    candidate knob set, pinned with ``tuning.table.override``, five warm-up and ten timed calls each,
    maximum over the ranks of the op's group - record the ranking, and install the winner in the
    run-time table so that later calls use it (reference: the per-op ``profiling`` methods iterate
    every registered hparams set the same way, src/gemm_rs/ths_op/gemm_reduce_scatter.cc:979-1060)."""
    out = fn()
    if prof_ctx is None or not torch.cuda.is_available():
        return out
    group = getattr(op, "pg", None)
    if key is None:
        prof_ctx.add(TuningRecord(name, {}, {}, time_cuda(fn, group=group)))
        return out
    from .table import candidates, load_tuning_record, override
    ranked = []
    for knobs in candidates(*key, segmented_rows=segmented_rows):
        with override(key, knobs):
            ms = time_cuda(fn, group=group)
        if hasattr(op, "check_status"):
            op.check_status()
        ranked.append((ms, knobs))
    ranked.sort(key=lambda r: r[0])
    best_ms, best = ranked[0]
    prof_ctx.add(TuningRecord(name, {"m": key[0], "n": key[1], "k": key[2],
                                     "top": [dict(k, ms=round(ms, 5)) for ms, k in ranked[:5]]}, best, best_ms))
    load_tuning_record({"key": list(key), "best": best})
    return fn()


def profile_dense_plain(op, input, weight, bias, output_buf, input_scale, weight_scale,
                        prof_ctx: Optional[ProfilingContext]):
    from ..ops import _dense
    from ..ops.gemm_only import as_nk
    w = as_nk(weight, op.transpose_weight)
    out = output_buf if output_buf is not None else torch.empty(
        (input.shape[0], w.shape[0]), dtype=op.output_dtype, device=input.device)
    from .table import candidates
    ranked = []
    for knobs in candidates(input.shape[0], w.shape[0], w.shape[1]):
        ms = time_cuda(lambda: _dense.plain_gemm(input, w, out, bias, input_scale, weight_scale, **knobs))
        ranked.append((ms, knobs))
    ranked.sort(key=lambda r: r[0])
    if prof_ctx is not None:
        prof_ctx.add(TuningRecord("gemm_only", {"m": input.shape[0], "n": w.shape[0], "k": w.shape[1],
                                                "top": [dict(k, ms=round(ms, 5)) for ms, k in ranked[:5]]},
                                  ranked[0][1], ranked[0][0]))
    _dense.plain_gemm(input, w, out, bias, input_scale, weight_scale, **ranked[0][1])
    return out
