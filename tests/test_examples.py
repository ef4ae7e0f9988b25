"""Builds the C++ examples against the public headers and the shared library and runs them on the host simulator
(ranks are threads of one process)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
EXAMPLES = [
    ("01_communicators/root_info_threads.cc", ["4"]),
    ("03_op_dev/mesh_send_recv.cc", ["4"]),
    ("03_op_dev/mesh_send_recv.cc", ["2"]),
    ("04_team_one_sided/team_signal_put.cc", ["4"]),
    ("04_team_one_sided/team_signal_put.cc", ["2"]),
    ("05_resources/reduce_scatter_primitives.cc", ["4"]),
    ("05_resources/reduce_scatter_primitives.cc", ["3"]),
]


@pytest.fixture(scope="module")
def library():
    import hcomm_b200
    hcomm_b200.load_library()
    return ROOT / "hcomm_b200" / "lib"


@pytest.mark.parametrize("src,args", EXAMPLES)
def test_example_runs_on_the_simulator(src, args, library, tmp_path):
    exe = tmp_path / (Path(src).stem + "_" + "_".join(args))
    cmd = ["g++", "-std=c++17", "-O1", "-pthread", f"-I{ROOT / 'include'}", str(ROOT / "examples" / src), "-o", str(exe),
           f"-L{library}", "-lhcomm", f"-Wl,-rpath,{library}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    env = dict(os.environ, HCCL_SIM="1", HCCL_BUFFSIZE="2", HCCL_EXEC_TIMEOUT="20")
    run = subprocess.run([str(exe), *args], capture_output=True, text=True, env=env, timeout=120)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert " ok" in run.stdout
