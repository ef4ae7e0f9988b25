"""Builds tests/api_sweep.cc against the public headers and runs it on the host simulator: the exported entry points
that the scenario tests do not reach, called from ranks that are threads of one process."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def sweep(tmp_path_factory):
    import hcomm_b200
    hcomm_b200.load_library()
    libdir = ROOT / "hcomm_b200" / "lib"
    name = "hcomm_cov" if os.environ.get("HCOMM_LIBRARY") == "cov" else "hcomm"      # the coverage run links that build
    exe = tmp_path_factory.mktemp("sweep") / "api_sweep"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "api_sweep.cc"), "-o", str(exe),
           f"-L{libdir}", "-l" + name, "-ldl", "-rdynamic", f"-Wl,-rpath,{libdir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-6000:]
    return exe


@pytest.mark.parametrize("ranks", [4, 3, 1])
def test_api_sweep_on_the_simulator(sweep, ranks):
    env = dict(os.environ, HCCL_SIM="1", HCCL_BUFFSIZE="2", HCCL_EXEC_TIMEOUT="20")
    run = subprocess.run([str(sweep), str(ranks)], capture_output=True, text=True, env=env, timeout=180)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-6000:]
    assert f"{ranks} ranks ok" in run.stdout
