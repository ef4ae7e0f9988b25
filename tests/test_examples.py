"""Builds the C++ examples against the public headers and the shared library and runs them on the host simulator
(ranks are threads of one process)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
EXAMPLES = [
    ("01_communicators/root_info_threads.cc", ["4"]),
    ("01_communicators/root_info_processes.cc", ["3"]),
    ("01_communicators/rank_table_processes.cc", ["3"]),
    ("01_communicators/init_all_one_process.cc", ["4"]),
    ("03_op_dev/mesh_send_recv.cc", ["4"]),
    ("03_op_dev/mesh_send_recv.cc", ["2"]),
    ("04_team_one_sided/team_signal_put.cc", ["4"]),
    ("04_team_one_sided/team_signal_put.cc", ["2"]),
    ("05_resources/reduce_scatter_primitives.cc", ["4"]),
    ("05_resources/reduce_scatter_primitives.cc", ["3"]),
    ("06_recovery/survivors_go_on.cc", ["4"]),
    ("07_messages/plan_exchange.cc", ["4"]),
    ("07_messages/plan_exchange.cc", ["2"]),
]


@pytest.fixture(scope="module")
def library():
    import hcomm_b200
    hcomm_b200.load_library()
    return ROOT / "hcomm_b200" / "lib"


@pytest.mark.parametrize("src,args", EXAMPLES)
def test_example_runs_on_the_simulator(src, args, library, tmp_path):
    exe = tmp_path / (Path(src).stem + "_" + "_".join(args))
    # HCOMM_LIBRARY=cov (the coverage run of hcomm_b200.utils.coverage) links the examples to that build of the library
    name = "hcomm_cov" if os.environ.get("HCOMM_LIBRARY") == "cov" else "hcomm"
    cmd = ["g++", "-std=c++17", "-O1", "-pthread", f"-I{ROOT / 'include'}", str(ROOT / "examples" / src), "-o", str(exe),
           f"-L{library}", "-l" + name, f"-Wl,-rpath,{library}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    env = dict(os.environ, HCCL_SIM="1", HCCL_BUFFSIZE="2", HCCL_EXEC_TIMEOUT="20")
    run = subprocess.run([str(exe), *args], capture_output=True, text=True, env=env, timeout=120)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert " ok" in run.stdout


@pytest.mark.gpu
def test_user_kernel_on_the_device_side_channel_api(library, tmp_path):
    """examples/03_op_dev/sm_engine_ring.cu: a user's CUDA kernel built against include/hcomm_device.cuh.  Compiled for
    sm_100a always; run with one rank per GPU when the box has at least two GPUs (its kernels wait for each other, so
    ranks never share a GPU)."""
    import torch
    exe = tmp_path / "sm_engine_ring"
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", f"-I{ROOT / 'include'}",
           str(ROOT / "examples" / "03_op_dev" / "sm_engine_ring.cu"), "-o", str(exe), f"-L{library}", "-lhcomm", "-Xlinker", f"-rpath={library}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    env = dict(os.environ, HCCL_EXEC_TIMEOUT="20", HCCL_BUFFSIZE="8")
    run = subprocess.run([str(exe), "2"], capture_output=True, text=True, env=env, timeout=180)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    if torch.cuda.device_count() >= 2:
        assert "2 ranks ok" in run.stdout
    else:
        assert "skipped" in run.stdout
