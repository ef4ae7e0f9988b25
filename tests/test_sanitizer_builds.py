"""The AddressSanitizer, ThreadSanitizer and UndefinedBehaviorSanitizer builds of the host runtime
(``python -m hcomm_b200.build --asan`` / ``--tsan`` / ``--ubsan``) under the simulator platform.

Skipped when the library has not been built.  Every scenario runs as separate processes with the sanitizer's runtime
preloaded; an address report of any kind, or a data race, fails the test."""
import subprocess
from pathlib import Path

import pytest

from mp_launch import launch

LIBDIR = Path(__file__).resolve().parent.parent / "hcomm_b200" / "lib"
needs_asan = pytest.mark.skipif(not (LIBDIR / "libhcomm_asan.so").exists(), reason="libhcomm_asan.so not built (python -m hcomm_b200.build --asan)")
needs_ubsan = pytest.mark.skipif(not (LIBDIR / "libhcomm_ubsan.so").exists(), reason="libhcomm_ubsan.so not built (python -m hcomm_b200.build --ubsan)")
needs_tsan = pytest.mark.skipif(not (LIBDIR / "libhcomm_tsan.so").exists(), reason="libhcomm_tsan.so not built (python -m hcomm_b200.build --tsan)")

SCENARIOS = [
    ("collectives", 3, {}),
    ("forced_algos", 3, {}),
    ("lifecycle", 2, {}),
    ("hcom", 3, {}),
    ("op_retry", 3, {"HCCL_OP_RETRY_ENABLE": "1", "HCCL_OP_RETRY_PARAMS": "MaxCnt:2,HoldTime:300,IntervalTime:100", "HCCL_EXEC_TIMEOUT": "6"}),
]
# the heartbeat thread and the ring monitor beside the descriptor-accept thread, with ranks that vanish or fall silent
MONITOR_SCENARIOS = [
    ("ring_monitor", 5, {"HCCL_HEARTBEAT_INTERVAL_MS": "100", "HCCL_HEARTBEAT_LOST_MS": "8000"}),
    ("silent_rank", 3, {"HCCL_HEARTBEAT_INTERVAL_MS": "100", "HCCL_HEARTBEAT_LOST_MS": "1500"}),
]


def _asan_env(extra=None):
    runtime = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not Path(runtime).exists():
        pytest.skip("the compiler's libasan.so was not found")
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_LIBRARY": "asan", "LD_PRELOAD": runtime,
           "ASAN_OPTIONS": "detect_leaks=0:exitcode=77"}          # the interpreter itself leaks by design
    env.update(extra or {})
    return env


@needs_asan
@pytest.mark.parametrize("scenario,world,extra", SCENARIOS + MONITOR_SCENARIOS)
def test_simulator_scenarios_are_clean_under_address_sanitizer(scenario, world, extra):
    codes, outs = launch(scenario, world, _asan_env(extra), timeout=300)
    text = "\n".join(outs)
    assert "AddressSanitizer" not in text, text[-4000:]
    assert codes == [0] * world, text[-4000:]


def _tsan_env(extra=None):
    runtime = subprocess.run(["g++", "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not Path(runtime).exists():
        pytest.skip("the compiler's libtsan.so was not found")
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_LIBRARY": "tsan", "LD_PRELOAD": runtime,
           "TSAN_OPTIONS": "exitcode=0 report_signal_unsafe=0 report_thread_leaks=0"}
    env.update(extra or {})
    return env


@needs_tsan
@pytest.mark.parametrize("scenario,world,extra", SCENARIOS + MONITOR_SCENARIOS)
def test_simulator_scenarios_have_no_data_race_under_thread_sanitizer(scenario, world, extra):
    # agents, reader threads, heartbeats, retry rounds and the simulator's stream workers all run in these scenarios
    codes, outs = launch(scenario, world, _tsan_env(extra), timeout=600)
    text = "\n".join(outs)
    assert "ThreadSanitizer: data race" not in text and "ThreadSanitizer: lock-order-inversion" not in text, text[-6000:]
    assert codes == [0] * world, text[-4000:]


@needs_ubsan
@pytest.mark.parametrize("scenario,world,extra", SCENARIOS[:3])
def test_simulator_scenarios_have_no_undefined_behaviour(scenario, world, extra):
    runtime = subprocess.run(["g++", "-print-file-name=libubsan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not Path(runtime).exists():
        pytest.skip("the compiler's libubsan.so was not found")
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_LIBRARY": "ubsan", "LD_PRELOAD": runtime, "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=0"}
    env.update(extra)
    codes, outs = launch(scenario, world, env, timeout=300)
    text = "\n".join(outs)
    assert "runtime error" not in text, text[-4000:]
    assert codes == [0] * world, text[-4000:]
