"""Line coverage of the host runtime under the CPU tests (the counterpart of the reference's ``build.sh --cov``,
build.sh:22-23,40).

``python -m hcomm_b200.utils.coverage [--report-only] [--markdown] [pytest arguments]`` builds ``libhcomm_cov.so``
(gcov counters in every host translation unit and in the host side of the ``.cu`` files), runs the tests that need no GPU
with ``HCOMM_LIBRARY=cov`` so that every rank process loads that library, and turns the counters that the processes left
beside the objects into one table: source file, executable lines, lines run, per cent.  Ranks that a scenario ends with
``os._exit`` leave no counters; what they ran is counted through their peers only.  Device code is not instrumented.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from collections import defaultdict
from pathlib import Path

from .. import build as _build

OBJDIR = _build.BUILD / "obj-cov"

# Tests that load the PyTorch extension are left out: it is linked against the plain library, and two copies of the
# runtime in one process would not share their registries.
DESELECT = ["--deselect", "tests/test_multiprocess_sim.py::test_torch_backend_operators_on_the_simulator",
            "--deselect", "tests/test_multiprocess_sim.py::test_ddp_with_fused_scale_hook_matches_local_mean_gradient",
            "--ignore", "tests/test_sanitizer_builds.py", "--ignore", "tests/test_models.py"]


def clear_counters() -> None:
    for p in OBJDIR.glob("*.gcda"):
        p.unlink()


def run_tests(extra) -> int:
    env = dict(os.environ, HCOMM_LIBRARY="cov")
    cmd = [sys.executable, "-m", "pytest", "tests", "-q", "-m", "not gpu", "-p", "no:cacheprovider", *DESELECT, *extra]
    return subprocess.run(cmd, cwd=_build.ROOT, env=env).returncode


def collect() -> dict:
    """source path relative to the repository -> {line: hits} summed over all translation units that contain the line."""
    lines = defaultdict(lambda: defaultdict(int))
    for gcda in sorted(OBJDIR.glob("*.gcda")):
        res = subprocess.run(["gcov", "--json-format", "--stdout", "-o", str(OBJDIR), str(gcda)], capture_output=True, text=True, cwd=OBJDIR)
        if res.returncode != 0:
            continue
        for doc in res.stdout.splitlines():
            doc = doc.strip()
            if not doc.startswith("{"):
                continue
            for f in json.loads(doc).get("files", []):
                path = Path(f["file"])
                if not path.is_absolute():
                    path = (OBJDIR / path).resolve()
                try:
                    rel = path.resolve().relative_to(_build.ROOT)
                except ValueError:
                    continue                      # system and CUDA headers
                if rel.parts[0] not in ("csrc", "include"):
                    continue
                for ln in f["lines"]:
                    lines[str(rel)][ln["line_number"]] += ln["count"]
    return lines


def table(lines: dict, markdown: bool = False) -> str:
    rows, tot, hit = [], 0, 0
    for path in sorted(lines):
        n = len(lines[path])
        h = sum(1 for c in lines[path].values() if c > 0)
        if n == 0:
            continue
        rows.append((path, n, h, 100.0 * h / n))
        tot += n
        hit += h
    rows.append(("total", tot, hit, 100.0 * hit / max(tot, 1)))
    if markdown:
        out = ["| source | lines | run | % |", "|---|---:|---:|---:|"]
        out += [f"| `{p}` | {n} | {h} | {pc:.1f} |" for p, n, h, pc in rows]
    else:
        w = max(len(r[0]) for r in rows)
        out = [f"{p:<{w}}  {n:>6}  {h:>6}  {pc:5.1f}" for p, n, h, pc in rows]
    return "\n".join(out)


def uncovered_functions(limit: int = 40):
    """(source, function) pairs that never ran, from gcov's function records; exported entry points first."""
    never = set()
    ran = set()
    for gcda in sorted(OBJDIR.glob("*.gcda")):
        res = subprocess.run(["gcov", "--json-format", "--stdout", "-o", str(OBJDIR), str(gcda)], capture_output=True, text=True, cwd=OBJDIR)
        for doc in res.stdout.splitlines():
            if not doc.strip().startswith("{"):
                continue
            for f in json.loads(doc).get("files", []):
                if "/csrc/" not in f["file"] and not f["file"].startswith("csrc"):
                    continue
                for fn in f.get("functions", []):
                    key = (Path(f["file"]).name, fn.get("demangled_name", fn["name"]))
                    (ran if fn["execution_count"] > 0 else never).add(key)
    out = sorted(never - ran, key=lambda k: (not k[1].startswith(("Hccl", "Hcom")), k))
    return out[:limit] if limit else out


def main(argv) -> int:
    report_only = "--report-only" in argv
    markdown = "--markdown" in argv
    functions = "--functions" in argv
    extra = [a for a in argv if a not in ("--report-only", "--markdown", "--functions")]
    rc = 0
    if not report_only:
        _build.build_core(cov=True)
        clear_counters()
        rc = run_tests(extra)
    print(table(collect(), markdown))
    if functions:
        print()
        for src, fn in uncovered_functions(0):
            print(f"never ran: {src}: {fn}")
    return rc


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
