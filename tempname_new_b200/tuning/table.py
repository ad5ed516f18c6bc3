"""Tile / raster choices of the dense tcgen05 kernel per problem shape.

The reference keeps one compiled-in C++ record per (meta, shape) under
``src/*/tuning_config/*.cu`` and can load more from ``FLUX_TUNE_CONFIG_FILE``; here the kernel
has three run-time knobs — CTA pairing (``cta_group``), tile width (``tile_n``) and the raster
group (``group_m``) — so the table is a small dict of measured winners plus a heuristic for
unseen shapes. ``python -m tempname_new_b200.tuning.tune_dense`` measures a shape and prints
the entry to add; ``FLUXB_TUNE_FILE`` names a JSON file of extra entries.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Tuple

Key = Tuple[int, int, int]

# (M rows computed per GPU, N, K) -> knobs. Measured on B200 (148 SMs, 1000 W cap), bf16, with
# `tune_dense --seconds 0.6` (back-to-back launches, so the power cap decides): TFLOP/s of the winner
# and of torch.matmul on the same box in the same process.
DENSE_TABLE: Dict[Key, Dict[str, int]] = {
    # 512 x 256 CTA-pair tiles (two MMAs per k-step share one B tile) win every large shape; the raster
    # group differs: 8 tile rows (4096 rows) unless N is small next to K
    (8192, 49152, 12288): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},   # 1358 | 1400
    (8192, 12288, 49152): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 4},   # 1354 | 1291
    (8192, 24576, 12288): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},   # 1354 | 1388
    (8192, 12288, 24576): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},   # 1333 | 1305
    (8192, 12288, 12288): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},   # 1323 | 1313
    (8192, 6144, 12288): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},    # 1267 | 1316
    (8192, 12288, 6144): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},    # 1291 | 1316
    (4096, 4096, 4096): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},     # 1176 | 1268
    (4096, 12288, 4096): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},    # 1229 | 1295
    (16384, 3584, 8192): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 2},    # 1255 | 1272
    (16384, 8192, 3584): {"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": 8},    # 1279 | 1371
}

_NUM_SMS = 148


def _wave_eff(tiles: int, slots: int) -> float:
    waves = -(-tiles // slots)
    return tiles / (waves * slots)


def heuristic(m: int, n: int, k: int, elt: int = 2) -> Dict[str, int]:
    """CTA pairs on 256 x 256 tiles unless the problem is too small to fill 74 pairs; raster groups
    of 2048 rows (with wave-synchronous tile starts the grid walks K together, so the group does
    not have to fit L2 over the whole K extent)."""
    if m >= 256 and n >= 256 and (m // 256) * -(-n // 256) >= _NUM_SMS // 4:
        cg, bn = 2, 256      # (tile_m stays 0: the launcher picks 512-row tiles when the rows allow them)
    elif n % 256 == 0 or n > 2048:
        cg, bn = 1, 256
    else:
        cg, bn = 1, 128
    group = 8 if cg == 2 else 16
    return {"cta_group": cg, "tile_n": bn, "group_m": group}


def candidates(m: int, n: int, k: int, elt: int = 2, segmented_rows: int = 0):
    """Knob sets worth timing for a dense-kernel problem: 512-row CTA-pair tiles (two MMAs share a B
    tile) where the rows allow them, 256-row CTA pairs, single CTAs; a few raster groups each.
    ``segmented_rows``: rows per rank segment of a fused op (0: plain GEMM over m rows)."""
    rows = segmented_rows or m
    out = []
    if rows >= 512 and n >= 256:
        out += [{"cta_group": 2, "tile_n": 256, "tile_m": 512, "group_m": g} for g in (2, 4, 8)]
    if rows >= 256 and n >= 256:
        out += [{"cta_group": 2, "tile_n": 256, "tile_m": 256, "group_m": g} for g in (4, 8)]
    out += [{"cta_group": 1, "tile_n": 256 if n >= 256 else 128, "tile_m": 128, "group_m": g} for g in (8, 16)]
    if n % 256:
        out.append({"cta_group": 1, "tile_n": 128, "tile_m": 128, "group_m": 16})
    return out


def _load_extra() -> Dict[Key, Dict[str, int]]:
    path = os.environ.get("FLUXB_TUNE_FILE")
    if not path:
        return {}
    with open(path) as f:
        raw = json.load(f)
    return {tuple(e["key"]): e["best"] for e in raw}


_EXTRA = None
_OVERRIDE: Dict[Key, Dict[str, int]] = {}


class override:
    """``with override((m, n, k), knobs):`` pins the knobs of one shape for the calls inside the
    block - how the tuners try candidates through the public ops."""

    def __init__(self, key: Key, knobs: Dict[str, int]):
        self.key, self.knobs = tuple(key), dict(knobs)

    def __enter__(self):
        self.prev = _OVERRIDE.get(self.key)
        _OVERRIDE[self.key] = self.knobs
        return self

    def __exit__(self, *exc):
        if self.prev is None:
            _OVERRIDE.pop(self.key, None)
        else:
            _OVERRIDE[self.key] = self.prev
        return False


def lookup(m: int, n: int, k: int, elt: int = 2) -> Dict[str, int]:
    global _EXTRA
    if _EXTRA is None:
        _EXTRA = _load_extra()
    key = (m, n, k)
    if key in _OVERRIDE:
        return dict(_OVERRIDE[key])
    if key in _EXTRA:
        return dict(_EXTRA[key])
    if key in DENSE_TABLE:
        return dict(DENSE_TABLE[key])
    return heuristic(m, n, k, elt)
