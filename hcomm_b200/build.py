"""In-tree build of the native parts.

Produces, under ``hcomm_b200/lib``:

* ``libhcomm.so``  - the communication library (C ABI of ``include/``): host runtime compiled with
  g++, every ``.cu`` compiled by nvcc for ``sm_100a`` only, CUDA runtime linked statically, no link
  against libcuda (driver entry points are resolved at run time) so the library also loads on a host
  without a GPU, where only the simulator platform is available.
* ``_hcomm_torch.so`` - the PyTorch extension (c10d backend and the fused operators), built on demand
  by :func:`build_torch_extension`.

Objects are cached in ``build/`` and recompiled when a source or any header is newer.
Run ``python -m hcomm_b200.build`` to build everything.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT / "include"
BUILD = ROOT / "build"
LIBDIR = ROOT / "hcomm_b200" / "lib"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-fvisibility=default",
             f"-I{INCLUDE}", f"-I{CUDA_HOME / 'include'}", "-pthread"]
NVCC_FLAGS = ARCH_FLAGS + ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", f"-I{INCLUDE}",
                           "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]

# Sources that belong to the torch extension rather than to libhcomm.so.
TORCH_DIR = CSRC / "torch"


def _headers_mtime() -> float:
    newest = 0.0
    for pattern in ("*.h", "*.cuh", "*.hpp"):
        for base in (CSRC, INCLUDE):
            for p in base.rglob(pattern):
                newest = max(newest, p.stat().st_mtime)
    return newest


def _core_sources():
    srcs = []
    for p in sorted(CSRC.rglob("*.cc")) + sorted(CSRC.rglob("*.cu")):
        if TORCH_DIR in p.parents:
            continue
        srcs.append(p)
    return srcs


def _obj_for(src: Path, variant: str = "") -> Path:
    rel = src.relative_to(CSRC)
    return BUILD / ("obj" + ("-" + variant if variant else "")) / (str(rel).replace("/", "__") + ".o")


ASAN_HOST_FLAGS = ["-fsanitize=address", "-fno-omit-frame-pointer", "-g"]
TSAN_HOST_FLAGS = ["-fsanitize=thread", "-fno-omit-frame-pointer", "-g"]
UBSAN_HOST_FLAGS = ["-fsanitize=undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g"]
COV_HOST_FLAGS = ["--coverage", "-O0", "-g", "-fprofile-update=atomic"]      # gcov counters, updated atomically (many threads)


def _compile(src: Path, hdr_mtime: float, verbose: bool, extra_nvcc=(), variant: str = "", defines=()) -> Path:
    obj = _obj_for(src, variant)
    obj.parent.mkdir(parents=True, exist_ok=True)
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_mtime):
        return obj
    san = {"asan": ASAN_HOST_FLAGS, "tsan": TSAN_HOST_FLAGS, "ubsan": UBSAN_HOST_FLAGS, "cov": COV_HOST_FLAGS}.get(variant, [])
    if src.suffix == ".cu":
        host = ["-Xcompiler", ",".join(san)] if san else []       # host side of the file only; device code has no such tool
        cmd = [NVCC, *NVCC_FLAGS, *extra_nvcc, *host, *defines, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, *san, *defines, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, file=sys.stderr)
    return obj


def build_core(verbose: bool = False, jobs: int | None = None, bounds: bool = False, asan: bool = False, tsan: bool = False, ubsan: bool = False,
               cov: bool = False) -> Path:
    """Builds ``libhcomm.so`` and returns its path.

    ``asan=True`` builds ``libhcomm_asan.so``: the host runtime (and the host side of the ``.cu`` files) compiled with
    AddressSanitizer.  Load it with ``HCOMM_LIBRARY=asan`` in a process started with ``LD_PRELOAD`` set to the compiler's
    ``libasan.so`` (``g++ -print-file-name=libasan.so``) and ``ASAN_OPTIONS=detect_leaks=0`` (the interpreter leaks by design);
    the simulator platform (``HCCL_SIM=1``) then runs the control plane, the host engine and the schedule interpreter under it.
    ``tsan=True`` builds ``libhcomm_tsan.so`` the same way with ThreadSanitizer (``HCOMM_LIBRARY=tsan``, preload ``libtsan.so``).

    ``cov=True`` builds ``libhcomm_cov.so`` with gcov counters in the host code (``HCOMM_LIBRARY=cov``); the counters
    land beside the objects in ``build/obj-cov`` when a process exits, and ``python -m hcomm_b200.utils.coverage`` runs
    the CPU tests on that library and prints line coverage per source file.

    ``bounds=True`` builds ``libhcomm_bounds.so`` instead: the same library compiled with ``-DHCOMM_DEBUG_BOUNDS``, in
    which every grid copy and reduction of the collective kernels checks its address ranges against the symmetric heap
    and the CCL halves and records a violation in the status block instead of touching memory out of range.  Select it
    at run time with ``HCOMM_LIBRARY=bounds``."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    variant = "bounds" if bounds else "asan" if asan else "tsan" if tsan else "ubsan" if ubsan else "cov" if cov else ""
    out = LIBDIR / ("libhcomm_" + variant + ".so" if variant else "libhcomm.so")
    srcs = _core_sources()
    hdr = _headers_mtime()
    jobs = jobs or min(8, os.cpu_count() or 4)
    defines = ("-DHCOMM_DEBUG_BOUNDS",) if bounds else ()
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr, verbose, variant=variant, defines=defines), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if out.exists() and out.stat().st_mtime >= newest_obj:
        return out
    link = ["g++", "-shared", "-o", str(out), *map(str, objs), f"-L{CUDA_HOME / 'lib64'}", "-lcudart_static",
            "-lpthread", "-ldl", "-lrt"] + (["-fsanitize=address"] if asan else ["-fsanitize=thread"] if tsan else ["-fsanitize=undefined"] if ubsan else ["--coverage"] if cov else ["-Wl,--no-undefined"])
    if verbose:
        print(" ".join(link), flush=True)
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"linking libhcomm.so failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_torch_extension(verbose: bool = False) -> Path:
    """Builds the PyTorch extension against the installed torch and links it to libhcomm.so."""
    import torch
    from torch.utils import cpp_extension as ce

    core = build_core(verbose)
    out = LIBDIR / "_hcomm_torch.so"
    srcs = sorted(TORCH_DIR.glob("*.cpp")) + sorted(TORCH_DIR.glob("*.cu"))
    if not srcs:
        raise RuntimeError("no sources under csrc/torch")
    hdr = _headers_mtime()
    newest = max([s.stat().st_mtime for s in srcs] + [hdr, core.stat().st_mtime])
    if out.exists() and out.stat().st_mtime >= newest:
        return out
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{INCLUDE}", f"-I{CSRC}"]
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_hcomm_torch", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    objs = []

    def one(src: Path) -> Path:
        obj = BUILD / "obj_torch" / (src.name + ".o")
        obj.parent.mkdir(parents=True, exist_ok=True)
        if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr):
            return obj
        if src.suffix == ".cu":
            cmd = [NVCC, *ARCH_FLAGS, "-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                   *inc, *common, "-c", str(src), "-o", str(obj)]
        else:
            cmd = ["g++", "-std=c++17", "-O2", "-fPIC", *inc, *common, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{res.stdout[-4000:]}\n{res.stderr[-8000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(one, srcs))
    torch_lib = Path(torch.__file__).parent / "lib"
    link = ["g++", "-shared", "-o", str(out), *map(str, objs), f"-L{LIBDIR}", "-lhcomm", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu",
            "-lc10", "-ltorch_python", f"-L{CUDA_HOME / 'lib64'}", "-lcudart_static", "-lpthread", "-ldl", "-lrt",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    if (torch_lib / "libtorch_cuda.so").exists():
        link += ["-ltorch_cuda", "-lc10_cuda"]
    if verbose:
        print(" ".join(link), flush=True)
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"linking _hcomm_torch.so failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_all(verbose: bool = False) -> None:
    build_core(verbose)
    if any(TORCH_DIR.glob("*.cpp")) or any(TORCH_DIR.glob("*.cu")):
        build_torch_extension(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    if "--bounds" in sys.argv:
        build_core(verbose="-v" in sys.argv, bounds=True)
    if "--asan" in sys.argv:
        build_core(verbose="-v" in sys.argv, asan=True)
    if "--tsan" in sys.argv:
        build_core(verbose="-v" in sys.argv, tsan=True)
    if "--ubsan" in sys.argv:
        build_core(verbose="-v" in sys.argv, ubsan=True)
    if "--cov" in sys.argv:
        build_core(verbose="-v" in sys.argv, cov=True)
    print("built:", *sorted(p.name for p in LIBDIR.glob("*.so")))
