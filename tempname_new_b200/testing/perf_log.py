"""Benchmark records as JSON lines (reference: ``python/flux/testing/perf_db_helper.py``, which
prints a ``PerfResult`` or uploads it to a MySQL database; the upload has no counterpart here)."""
from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, Optional

import torch


@dataclass
class PerfResult:
    name: str
    output: Optional[torch.Tensor] = None
    total_ms: float = 0.0
    gemm_time_ms: float = 0.0
    comm_time_ms: float = 0.0
    extra: Dict = field(default_factory=dict)

    def __repr__(self) -> str:
        return (f"{self.name}: total {self.total_ms:.3f} ms, gemm {self.gemm_time_ms:.3f} ms, "
                f"comm {self.comm_time_ms:.3f} ms")


def log_perf(result: PerfResult, file=None) -> None:
    """One JSON line per result: to ``file``, else to ``$FLUXB_PERF_LOG`` when set, else stdout."""
    rec = {k: v for k, v in asdict(result).items() if k != "output"}
    rec["time"] = time.time()
    rec["device"] = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    line = json.dumps(rec)
    path = os.environ.get("FLUXB_PERF_LOG")
    if file is not None:
        file.write(line + "\n")
    elif path:
        with open(path, "a") as f:
            f.write(line + "\n")
    else:
        sys.stdout.write(line + "\n")


# ------------------------------------------------------------------------------------------
# names of the reference's perf database helper (python/flux/testing/perf_db_helper.py:135-386).
# The MySQL ("RDS") upload has no counterpart: there is no database on the other side, so the
# switch is always off and the upload says so.
# ------------------------------------------------------------------------------------------
def should_log_to_rds() -> bool:
    return False


def log_perf_stdout(result: PerfResult) -> None:
    print(result)


def upload_to_rds(result: PerfResult) -> None:
    raise NotImplementedError("no performance database is attached to this library; use log_perf "
                              "(JSON lines, FLUXB_PERF_LOG) instead")


def log_perf_rds(result: PerfResult) -> None:
    if should_log_to_rds():
        upload_to_rds(result)


def query(delete: bool = False):
    """Records written so far to ``$FLUXB_PERF_LOG`` (the reference queries its database);
    ``delete`` empties the file."""
    path = os.environ.get("FLUXB_PERF_LOG")
    if not path or not os.path.exists(path):
        return []
    with open(path) as f:
        recs = [json.loads(line) for line in f if line.strip()]
    if delete:
        open(path, "w").close()
    return recs
