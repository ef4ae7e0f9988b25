"""Static verification of every algorithm template: semantics, notify balance, deadlock freedom and
memory conflicts (the role of the reference's task-DAG checker), plus proof that the checker notices
broken schedules."""
import pytest

from simutil import CMD, tool_str


def _lib():
    from hcomm_b200 import _lib
    return _lib.load()


@pytest.mark.parametrize("cmd", ["allreduce", "reducescatter", "allgather", "alltoall", "broadcast", "reduce", "scatter", "gather"])
def test_every_template_verifies(cmd):
    lib = _lib()
    checked = 0
    for n in range(1, 10):
        _, algos = tool_str(lib.HcommToolListAlgos, CMD[cmd], n)
        for algo in algos.split(","):
            for root in sorted({0, n - 1}):
                for inplace in ((0, 1) if cmd in ("allreduce", "broadcast") else (0,)):
                    rc, rep = tool_str(lib.HcommToolCheckSchedule, CMD[cmd], n, algo.encode(), 1000 + n, root, inplace, 0)
                    assert rc == 0, rep
                    checked += 1
    assert checked >= 17


def test_send_recv_template():
    rc, rep = tool_str(_lib().HcommToolCheckSchedule, CMD["send"], 4, b"mesh", 100, 0, 0, 0)
    assert rc == 0, rep


@pytest.mark.parametrize("mutate,needle", [(1, ("conflict", "imbalance", "nobody has written", "semantics")), (2, ("deadlock", "imbalance")),
                                           (3, ("semantics", "conflict", "nobody has written"))])
@pytest.mark.parametrize("algo", [b"ring", b"mesh", b"H-D_R"])
def test_checker_catches_broken_schedules(mutate, needle, algo):
    rc, rep = tool_str(_lib().HcommToolCheckSchedule, CMD["allreduce"], 4, algo, 4096, 0, 0, mutate)
    assert rc == 1, rep
    assert any(k in rep for k in needle), rep


def test_unsupported_combinations_are_refused():
    rc, rep = tool_str(_lib().HcommToolCheckSchedule, CMD["reducescatter"], 6, b"H-D_R", 64, 0, 0, 0)
    assert rc == 2 and "power-of-two" in rep
    rc, rep = tool_str(_lib().HcommToolCheckSchedule, CMD["allgather"], 6, b"NB", 64, 0, 0, 0)
    assert rc == 0, rep   # Bruck serves any rank count


def test_schedule_dump_is_readable():
    rc, text = tool_str(_lib().HcommToolDumpSchedule, CMD["allreduce"], 4, b"ring", 1024, 0, 1)
    assert rc == 0 and "AllReduceRing rank 1/4" in text and "WRITE" in text and "WAIT" in text


def test_nhr_and_bruck_reduce_scatter_are_schedules_of_their_own():
    lib = _lib()
    for n in range(2, 9):
        for cmd, want in (("allreduce", "AllReduceNHR"), ("reducescatter", "ReduceScatterNHR"), ("allgather", "AllGatherNHR")):
            rc, text = tool_str(lib.HcommToolDumpSchedule, CMD[cmd], n, b"NHR", 4096, 0, n - 1)
            assert rc == 0 and want in text, text[:200]
            rc, rep = tool_str(lib.HcommToolCheckSchedule, CMD[cmd], n, b"NHR", 4096 + n, 0, 0, 0)
            assert rc == 0, rep
        rc, text = tool_str(lib.HcommToolDumpSchedule, CMD["reducescatter"], n, b"NB", 4096, 0, 0)
        assert rc == 0 and "ReduceScatterBruck" in text
    # log-step: an 8-rank NHR all-reduce has 3 + 3 exchange steps where the ring has 7 + 7
    _, nhr = tool_str(lib.HcommToolDumpSchedule, CMD["allreduce"], 8, b"NHR", 4096, 0, 0)
    _, ring = tool_str(lib.HcommToolDumpSchedule, CMD["allreduce"], 8, b"ring", 4096, 0, 0)
    assert nhr.count("WAIT") < ring.count("WAIT")
