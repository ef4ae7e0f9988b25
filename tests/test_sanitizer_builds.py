"""The AddressSanitizer, ThreadSanitizer and UndefinedBehaviorSanitizer builds of the host runtime
(``python -m hcomm_b200.build --asan`` / ``--tsan`` / ``--ubsan``) under the simulator platform.

Skipped when the library has not been built.  Every scenario runs as separate processes with the sanitizer's runtime
preloaded; an address report of any kind, or a data race, fails the test."""
import os
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
    ("peer_exit", 3, {}),                                  # the survivors derive a communicator from the old one
    ("peer_exit", 4, {"HCOMM_TEST_HUB_EXIT": "1"}),        # the hub's process is gone: the survivors start over among themselves
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


def _build_sweep(tmp_path, variant):
    """tests/api_sweep.cc linked against a sanitizer build of the library (with ThreadSanitizer the program is instrumented too)."""
    root = LIBDIR.parent.parent
    exe = tmp_path / ("api_sweep_" + variant)
    extra = ["-fsanitize=thread"] if variant == "tsan" else ["-Wl,--allow-shlib-undefined"]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread", f"-I{root / 'include'}", str(root / "tests" / "api_sweep.cc"), "-o", str(exe),
           f"-L{LIBDIR}", "-lhcomm_" + variant, "-ldl", "-rdynamic", f"-Wl,-rpath,{LIBDIR}", *extra]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-6000:]
    return exe


@needs_asan
def test_api_sweep_is_clean_under_address_sanitizer(tmp_path):
    exe = _build_sweep(tmp_path, "asan")
    env = dict(os.environ, **_asan_env({"HCCL_BUFFSIZE": "2", "HCCL_EXEC_TIMEOUT": "60"}))
    run = subprocess.run([str(exe), "4"], capture_output=True, text=True, env=env, timeout=300)
    text = run.stdout + run.stderr
    assert "AddressSanitizer" not in text, text[-6000:]
    assert run.returncode == 0 and "4 ranks ok" in run.stdout, text[-4000:]


@needs_tsan
def test_api_sweep_has_no_data_race_under_thread_sanitizer(tmp_path):
    # ranks are threads of one process here, so the registries, the control plane and the simulator's memory are shared
    exe = _build_sweep(tmp_path, "tsan")
    env = dict(os.environ, **_tsan_env({"HCCL_BUFFSIZE": "2", "HCCL_EXEC_TIMEOUT": "120"}))
    run = subprocess.run([str(exe), "4"], capture_output=True, text=True, env=env, timeout=600)
    text = run.stdout + run.stderr
    assert "ThreadSanitizer: data race" not in text and "ThreadSanitizer: lock-order-inversion" not in text, text[-8000:]
    assert run.returncode == 0 and "4 ranks ok" in run.stdout, text[-4000:]


@needs_asan
def test_parsers_survive_damaged_input_under_address_sanitizer():
    import sys
    env = dict(os.environ, **_asan_env())
    run = subprocess.run([sys.executable, str(Path(__file__).resolve().parent / "fuzz_parsers.py"), "4000", "23"], capture_output=True, text=True, errors="replace", env=env, timeout=900)
    text = run.stdout + run.stderr
    assert "AddressSanitizer" not in text, text[-6000:]
    assert run.returncode == 0 and "fuzz: 4000 inputs" in run.stdout, text[-4000:]


@needs_ubsan
def test_api_sweep_has_no_undefined_behaviour(tmp_path):
    runtime = subprocess.run(["g++", "-print-file-name=libubsan.so"], capture_output=True, text=True).stdout.strip()
    if not runtime or not Path(runtime).exists():
        pytest.skip("the compiler's libubsan.so was not found")
    exe = _build_sweep(tmp_path, "ubsan")
    env = dict(os.environ, HCCL_SIM="1", HCCL_BUFFSIZE="2", HCCL_EXEC_TIMEOUT="60", LD_PRELOAD=runtime, UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=0")
    run = subprocess.run([str(exe), "4"], capture_output=True, text=True, env=env, timeout=300)
    text = run.stdout + run.stderr
    assert "runtime error" not in text, text[-6000:]
    assert run.returncode == 0 and "4 ranks ok" in run.stdout, text[-4000:]


@needs_asan
def test_communicator_creation_survives_damaged_configuration_under_address_sanitizer():
    import sys
    env = dict(os.environ, **_asan_env())
    run = subprocess.run([sys.executable, str(Path(__file__).resolve().parent / "fuzz_config.py"), "150", "9"], capture_output=True, text=True, errors="replace", env=env, timeout=900)
    text = run.stdout + run.stderr
    assert "AddressSanitizer" not in text, text[-6000:]
    assert run.returncode == 0 and "config fuzz: 150 structures" in run.stdout, text[-4000:]
