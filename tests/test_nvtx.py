"""Operators are wrapped in NVTX ranges while profiling is on: checked with a small injection library that NVTX loads
in place of a profiler and that logs every range."""
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CUDA_INCLUDE = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"

CHILD = """
import sys, torch
sys.path.insert(0, %r)
import hcomm_b200 as hb
c = hb.Communicator(1, hb.get_root_info(), 0, buffer_mb=2)
x = torch.arange(1000, dtype=torch.float32)
y = torch.empty_like(x)
c.all_reduce(x, y)                                            # profiling off: no range
c.set_profiling(True)
c.all_reduce(x, y)
c.all_gather(x, y)
c.set_profiling(False)
assert c.kernel_times() == []                                 # the simulator runs no kernels
assert "allreduce" in c.dump().lower().replace("_", ""), c.dump()
c.all_reduce(x, y)
c.destroy()
""" % str(ROOT)


def test_profiled_operators_emit_one_nvtx_range_each(tmp_path):
    so = tmp_path / "libnvtx_injection.so"
    res = subprocess.run(["g++", "-shared", "-fPIC", "-O1", f"-I{CUDA_INCLUDE}", str(ROOT / "tests" / "nvtx_injection.cc"), "-o", str(so)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    log = tmp_path / "ranges.txt"
    env = dict(os.environ, HCCL_SIM="1", NVTX_INJECTION64_PATH=str(so), HC_NVTX_LOG=str(log))
    run = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=180)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    lines = log.read_text().splitlines()
    pushes = [ln for ln in lines if ln.startswith("push hccl:")]
    assert len(pushes) == 2 and lines.count("pop") == 2, lines
    assert "allreduce" in pushes[0].lower().replace("_", "") and "1000 x" in pushes[0]
    assert "allgather" in pushes[1].lower().replace("_", "")
    assert lines[0].startswith("push") and lines[1] == "pop"   # ranges do not nest: one per operator
