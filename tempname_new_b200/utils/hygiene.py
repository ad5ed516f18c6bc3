"""Source hygiene for this tree: ``python -m tempname_new_b200.utils.hygiene [--check] [--fix]``.

Checks every tracked source file (``.py .cu .cuh .cc .h .sh``) for tabs, trailing blanks, a missing
final newline and lines over 132 columns, checks that comments and docstrings stand on their own
(they must not point at working notes of a build, at a reviewer, or at paths of one machine), and
runs ``clang-format --dry-run`` / ``black --check`` when those tools are installed. ``--fix``
rewrites the whitespace problems in place. Exit code 1 when anything is left to fix.

Reference: ``code-format.sh`` (clang-format / black over the changed files), the ``pre-commit``
hook and ``tools/check_license.py`` of the reference tree; here one module does the three jobs and
``.pre-commit-config.yaml`` wires it into ``git commit``.
"""
from __future__ import annotations

import argparse
import re
import shutil
import subprocess
import sys
from pathlib import Path
from typing import Iterable, List, Tuple

ROOT = Path(__file__).resolve().parents[2]
SOURCE_SUFFIXES = {".py", ".cu", ".cuh", ".cc", ".h", ".sh"}
SKIP_DIRS = {".git", "build", "gpurun_out", "_work", "__pycache__", "baseline", ".pytest_cache"}
MAX_COLUMNS = 132

# words that tie a comment to one build of the tree instead of stating the fact itself
_STRAY = re.compile(
    r"\b(SURVEY|VERDICT|ADVICE|DESIGN|BASELINE)\.md\b|\bgpurun\b|/root/(repo|reference)\b|\bround [0-9]+\b",
    re.IGNORECASE)


def tracked_sources(root: Path = ROOT) -> List[Path]:
    try:
        out = subprocess.run(["git", "ls-files"], cwd=root, capture_output=True, text=True, check=True).stdout
        files = [root / line for line in out.splitlines() if line]
    except (OSError, subprocess.CalledProcessError):
        files = [p for p in root.rglob("*") if p.is_file() and not (set(p.relative_to(root).parts) & SKIP_DIRS)]
    return [f for f in files if f.suffix in SOURCE_SUFFIXES and f.exists()
            and not (set(f.relative_to(root).parts) & SKIP_DIRS)]


def check_text(path: Path, text: str) -> List[Tuple[int, str]]:
    """(line number, problem) pairs of one file."""
    problems = []
    lines = text.split("\n")
    for i, line in enumerate(lines, 1):
        if "\t" in line and path.suffix != ".sh":
            problems.append((i, "tab character"))
        if line != line.rstrip():
            problems.append((i, "trailing whitespace"))
        if len(line) > MAX_COLUMNS:
            problems.append((i, f"line longer than {MAX_COLUMNS} columns"))
        if path.name != "hygiene.py" and _STRAY.search(line):
            problems.append((i, "comment or string points outside the source tree"))
    if text and not text.endswith("\n"):
        problems.append((len(lines), "no newline at end of file"))
    return problems


def fix_text(text: str) -> str:
    lines = [line.rstrip() for line in text.split("\n")]
    while lines and lines[-1] == "":
        lines.pop()
    return "\n".join(lines) + "\n"


def run_formatters(files: Iterable[Path]) -> List[str]:
    """Messages of the external formatters that are installed (none installed: nothing to say)."""
    msgs = []
    files = list(files)
    cpp = [str(f) for f in files if f.suffix in {".cu", ".cuh", ".cc", ".h"}]
    py = [str(f) for f in files if f.suffix == ".py"]
    cf = shutil.which("clang-format")
    if cf and cpp:
        r = subprocess.run([cf, "--dry-run", "--Werror", *cpp], capture_output=True, text=True)
        if r.returncode != 0:
            msgs.append("clang-format: " + r.stderr.strip().splitlines()[0] if r.stderr.strip() else "clang-format failed")
    bl = shutil.which("black")
    if bl and py:
        r = subprocess.run([bl, "--check", "-q", *py], capture_output=True, text=True)
        if r.returncode != 0:
            msgs.append("black: files would be reformatted")
    return msgs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hygiene")
    ap.add_argument("--check", action="store_true", help="report only (default)")
    ap.add_argument("--fix", action="store_true", help="rewrite whitespace problems in place")
    ap.add_argument("--formatters", action="store_true", help="also run clang-format / black when installed")
    args = ap.parse_args(argv)
    bad = 0
    files = tracked_sources()
    for f in files:
        text = f.read_text(errors="replace")
        if args.fix:
            fixed = fix_text(text)
            if fixed != text:
                f.write_text(fixed)
                text = fixed
        for line, what in check_text(f, text):
            print(f"{f.relative_to(ROOT)}:{line}: {what}")
            bad += 1
    if args.formatters:
        for m in run_formatters(files):
            print(m)
            bad += 1
    print(f"{len(files)} files checked, {bad} problem(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
