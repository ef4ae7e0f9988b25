"""The AddressSanitizer build of the host runtime (``python -m hcomm_b200.build --asan``) under the simulator platform.

Skipped when ``libhcomm_asan.so`` has not been built.  Every scenario runs as separate processes with the sanitizer's runtime
preloaded; a report of any kind fails the test."""
import subprocess
from pathlib import Path

import pytest

from mp_launch import launch

LIB = Path(__file__).resolve().parent.parent / "hcomm_b200" / "lib" / "libhcomm_asan.so"
pytestmark = pytest.mark.skipif(not LIB.exists(), reason="libhcomm_asan.so not built (python -m hcomm_b200.build --asan)")


def _asan_env(extra=None):
    runtime = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not Path(runtime).exists():
        pytest.skip("the compiler's libasan.so was not found")
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_LIBRARY": "asan", "LD_PRELOAD": runtime,
           "ASAN_OPTIONS": "detect_leaks=0:exitcode=77"}          # the interpreter itself leaks by design
    env.update(extra or {})
    return env


@pytest.mark.parametrize("scenario,world,extra", [
    ("collectives", 3, {}),
    ("forced_algos", 3, {}),
    ("lifecycle", 2, {}),
    ("hcom", 3, {}),
    ("op_retry", 3, {"HCCL_OP_RETRY_ENABLE": "1", "HCCL_OP_RETRY_PARAMS": "MaxCnt:2,HoldTime:300,IntervalTime:100", "HCCL_EXEC_TIMEOUT": "4"}),
])
def test_simulator_scenarios_are_clean_under_address_sanitizer(scenario, world, extra):
    codes, outs = launch(scenario, world, _asan_env(extra), timeout=300)
    text = "\n".join(outs)
    assert "AddressSanitizer" not in text, text[-4000:]
    assert codes == [0] * world, text[-4000:]
