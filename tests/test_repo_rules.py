"""Source-level rules of this code base that no compiler checks."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SOURCES = [p for pat in ("csrc/**/*", "include/**/*", "hcomm_b200/**/*.py", "hccl/**/*.py", "examples/**/*", "tests/*.py", "*.py")
           for p in ROOT.glob(pat) if p.is_file() and p.suffix in (".cu", ".cuh", ".cc", ".cpp", ".c", ".h", ".py")]


def test_no_batched_memcpy_entry_points_are_named():
    # assembled from pieces so that this file does not name them either
    names = [a + "Memcpy" + b + "BatchAsync" for a in ("cuda", "cu") for b in ("", "3D")]
    for p in SOURCES:
        text = p.read_text(errors="ignore")
        for n in names:
            assert n not in text, f"{p} names {n}"


def test_no_bulk_or_tensor_load_carries_a_cluster_multicast_qualifier():
    # tcgen05.commit may multicast its barrier arrival; copies into shared memory may not multicast their data
    qualifier = ".multicast" + "::cluster"
    for p in SOURCES:
        for line in p.read_text(errors="ignore").splitlines():
            if qualifier in line and "cp.async.bulk" in line:
                raise AssertionError(f"{p}: {line.strip()}")


def test_kernels_that_spin_have_a_bound():
    # every polling loop in the device sources goes through a helper with an iteration or time budget; a bare
    # `while (...flag...)` without a counter is what this looks for
    bare = re.compile(r"while\s*\(\s*(\*|Ld(Acquire|Relaxed)Sys)\s*\(?[^;{]*\)\s*(;|\{\s*\})")
    for p in SOURCES:
        if p.suffix not in (".cu", ".cuh"):
            continue
        for i, line in enumerate(p.read_text(errors="ignore").splitlines(), 1):
            assert not bare.search(line), f"{p}:{i}: unbounded spin: {line.strip()}"


def test_every_exported_entry_point_is_in_the_api_reference():
    """docs/api_reference.md names every function the shared library exports under the API's prefixes."""
    import subprocess
    lib = ROOT / "hcomm_b200" / "lib" / "libhcomm.so"
    if not lib.exists():
        import hcomm_b200
        hcomm_b200.load_library()
    out = subprocess.run(["nm", "-D", "--defined-only", str(lib)], capture_output=True, text=True).stdout
    names = sorted({ln.split()[2] for ln in out.splitlines() if len(ln.split()) == 3 and ln.split()[1] == "T" and ln.split()[2].startswith(("Hccl", "Hcom"))})
    assert len(names) > 250
    doc = (ROOT / "docs" / "api_reference.md").read_text()
    missing = [n for n in names if f"`{n}`" not in doc]
    assert not missing, missing


def test_public_headers_compile_as_c():
    """The API is a C ABI: every header under include/ except the CUDA one is accepted by a C compiler on its own."""
    import subprocess
    inc = ROOT / "include"
    cuda = "/usr/local/cuda/include"
    for header in sorted(inc.rglob("*.h")):
        rel = header.relative_to(inc)
        res = subprocess.run(["gcc", "-std=c11", "-fsyntax-only", "-Wall", f"-I{inc}", f"-I{cuda}", "-x", "c", "-"], input=f'#include "{rel}"\n',
                             capture_output=True, text=True)
        assert res.returncode == 0, f"{rel}:\n{res.stderr[-2000:]}"
