"""Real multi-GPU runs: one process per GPU, peer memory mapped through exported VMM handles."""
import pytest

from conftest import cuda_device_count
from mp_launch import launch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_across_gpus(world):
    if cuda_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, outs = launch("collectives", world, {"HCOMM_TEST_BUFFER_MB": "16", "HCCL_EXEC_TIMEOUT": "20"}, timeout=150)
    assert codes == [0] * world, "\n".join(outs)


@pytest.mark.parametrize("world", [2, 8])
def test_windows_nvls_and_registered_buffers_across_gpus(world):
    if cuda_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, outs = launch("collectives_big", world, {"HCOMM_TEST_BUFFER_MB": "16", "HCCL_EXEC_TIMEOUT": "30", "HCCL_NVLS_PIPELINE_MIN_MB": "32"}, timeout=300)
    assert codes == [0] * world, "\n".join(outs)


def test_peer_exit_between_steps_is_seen_on_the_host():
    if cuda_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    codes, outs = launch("peer_exit", 2, {"HCOMM_TEST_BUFFER_MB": "8", "HCCL_NVLS_ENABLE": "0", "NCCL_NVLS_ENABLE": "0", "HCCL_EXEC_TIMEOUT": "20"}, timeout=90)
    assert codes[0] == 0, "\n".join(outs)


@pytest.mark.parametrize("world", [2, 8])
def test_fused_kernels_across_gpus(world):
    if cuda_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, outs = launch("fused", world, {"HCOMM_TEST_BUFFER_MB": "32", "HCCL_EXEC_TIMEOUT": "20"}, timeout=200)
    assert codes == [0] * world, "\n".join(outs)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_kernels_at_the_benchmark_shapes(world):
    if cuda_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, outs = launch("fused_bench_shapes", world, {"HCOMM_TEST_BUFFER_MB": "512", "HCCL_EXEC_TIMEOUT": "30"}, timeout=300)
    assert codes == [0] * world, "\n".join(outs)


@pytest.mark.parametrize("form", ["communication_ctas", "no_signaller", "signaller_everywhere"])
def test_fused_kernels_in_their_other_forms(form):
    # the same shapes with CTAs set aside for communication (all-gather pushers; reduce-scatter outbox and forwarders),
    # with every data-moving warp publishing its own tiles, and with a signaller warp in both kernels
    if cuda_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = {"communication_ctas": {"HCOMM_FUSED_COMM_CTAS": "16", "HCOMM_FUSED_RS_COMM_CTAS": "16"}, "no_signaller": {"HCOMM_FUSED_SIGNALLER": "0"},
             "signaller_everywhere": {"HCOMM_FUSED_SIGNALLER": "1"}}[form]
    codes, outs = launch("fused_bench_shapes", 2, {"HCOMM_TEST_BUFFER_MB": "512", "HCCL_EXEC_TIMEOUT": "30", **extra}, timeout=300)
    assert codes == [0, 0], "\n".join(outs)


@pytest.mark.parametrize("scenario", ["torch_ops", "torch_ddp"])
def test_torch_backend_across_gpus(scenario):
    if cuda_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"HCOMM_TORCH_BUFFER_MB": "16", "HCCL_EXEC_TIMEOUT": "20", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29651"}
    codes, outs = launch(scenario, 2, env, timeout=200)
    assert codes == [0, 0], "\n".join(outs)


def test_forced_algorithm_families_across_gpus():
    if cuda_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    codes, outs = launch("forced_algos", 2, {"HCOMM_TEST_BUFFER_MB": "8", "HCCL_EXEC_TIMEOUT": "20"}, timeout=200)
    assert codes == [0, 0], "\n".join(outs)


def test_all_reduce_in_a_captured_cuda_graph_across_gpus():
    """examples/02_graphs/allreduce_cuda_graph_demo.py on two GPUs: five replays of one captured all-reduce."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    if cuda_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29671",
           str(root / "examples" / "02_graphs" / "allreduce_cuda_graph_demo.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, HCCL_EXEC_TIMEOUT="20"))
    assert res.returncode == 0 and "5 replays ok" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
