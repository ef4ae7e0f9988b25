"""Every collective on the host simulator, ranks as threads of this process, checked against NumPy.

Includes the reference configuration "AllReduce sum, fp32, 1,048,576 elements per rank, 8 ranks
simulated in-process, inputs uniform[-1,1] from seed+rank, compared with the exact elementwise sum".
"""
import numpy as np
import pytest

from helpers import run_ranks
from simutil import destroy, make_comms, sim_env


def test_allreduce_8_ranks_1mi_fp32_exact_sum(monkeypatch):
    sim_env(monkeypatch, buffsize=8)
    n, count, seed = 8, 1 << 20, 2024
    comms = make_comms(n)
    xs = [np.random.default_rng(seed + r).uniform(-1, 1, count).astype(np.float32) for r in range(n)]
    outs = [np.empty_like(x) for x in xs]
    run_ranks(n, lambda r: comms[r].all_reduce(xs[r], outs[r]))
    # the library adds contributions in ascending rank order in fp32: reproduce exactly
    ref = xs[0].copy()
    for r in range(1, n):
        ref = ref + xs[r]
    for r in range(n):
        assert np.array_equal(outs[r], ref)
    assert np.abs(outs[0].astype(np.float64) - np.sum([x.astype(np.float64) for x in xs], axis=0)).max() < 1e-5
    destroy(comms)


@pytest.mark.parametrize("algo", ["", "level0:ring", "level0:H-D_R", "level0:NHR", "level0:fullmesh", "allreduce=level0:mesh_oneshot/others=level0:ring"])
@pytest.mark.parametrize("n", [2, 3, 5, 8])
def test_allreduce_algorithms(monkeypatch, algo, n):
    sim_env(monkeypatch, HCCL_ALGO=algo)
    comms = make_comms(n)
    for count, dt in ((1, np.float32), (1001, np.float64), (70000, np.int32), (333, np.float16)):
        xs = [np.random.default_rng(r).integers(-50, 50, count).astype(dt) for r in range(n)]
        outs = [np.empty_like(x) for x in xs]
        run_ranks(n, lambda r: comms[r].all_reduce(xs[r], outs[r]))
        ref = np.sum(xs, axis=0).astype(dt)
        for r in range(n):
            assert np.array_equal(outs[r], ref), (algo, n, count, dt)
    destroy(comms)


@pytest.mark.parametrize("op,fn", [("max", np.max), ("min", np.min), ("prod", np.prod)])
def test_allreduce_ops_in_place(monkeypatch, op, fn):
    sim_env(monkeypatch)
    n = 4
    comms = make_comms(n)
    xs = [np.random.default_rng(r).integers(1, 4, 5000).astype(np.int64) for r in range(n)]
    ref = fn(np.stack(xs), axis=0)
    bufs = [x.copy() for x in xs]
    run_ranks(n, lambda r: comms[r].all_reduce(bufs[r], None, op=op))
    for r in range(n):
        assert np.array_equal(bufs[r], ref)
    destroy(comms)


@pytest.mark.parametrize("algo", ["", "level0:ring", "level0:NB", "level0:NHR", "level0:pairwise"])
@pytest.mark.parametrize("n", [1, 4, 7])
def test_all_collectives(monkeypatch, algo, n):
    sim_env(monkeypatch, HCCL_ALGO=algo)
    import hcomm_b200 as hb
    comms = make_comms(n)
    out = {}

    def body(r):
        c = comms[r]
        rng = np.random.default_rng(r)
        d = {}
        d["x"] = rng.normal(size=1000).astype(np.float32); d["y"] = np.zeros(1000 * n, np.float32); c.all_gather(d["x"], d["y"])
        d["a"] = rng.normal(size=777 * n).astype(np.float32); d["b"] = np.zeros(777, np.float32); c.reduce_scatter(d["a"], d["b"])
        d["s"] = (np.arange(n * 300) + r * 100000).astype(np.int32); d["t"] = np.zeros(n * 300, np.int32); c.all_to_all(d["s"], d["t"])
        d["z"] = np.full(5000, r, np.int64); c.broadcast(d["z"], root=n - 1)
        d["ri"] = rng.integers(0, 100, 3333).astype(np.int32); d["ro"] = np.zeros(3333, np.int32); c.reduce(d["ri"], d["ro"], root=1 % n, op="max")
        d["big"] = rng.uniform(-1, 1, 700000).astype(np.float32); d["bo"] = np.zeros_like(d["big"]); c.all_reduce(d["big"], d["bo"])
        d["sc_in"] = (np.arange(50 * n) + 1000 * r).astype(np.float32); d["sc_out"] = np.zeros(50, np.float32); c.scatter(d["sc_in"], d["sc_out"], root=0)
        d["g_out"] = np.zeros(50 * n, np.float32); c.gather(d["sc_out"], d["g_out"], root=n - 1)
        sc = [(r + q) % 3 * 10 + 5 for q in range(n)]; rc = [(q + r) % 3 * 10 + 5 for q in range(n)]
        sd = np.cumsum([0] + sc[:-1]).tolist(); rd = np.cumsum([0] + rc[:-1]).tolist()
        d.update(sc=sc, rc=rc, sd=sd, rd=rd)
        d["sv"] = (np.arange(sum(sc)) + 1000 * r).astype(np.float32); d["rv"] = np.zeros(sum(rc), np.float32)
        c.all_to_all_v(d["sv"], sc, sd, d["rv"], rc, rd)
        cnts = [10 + 3 * q for q in range(n)]; dsp = np.cumsum([0] + cnts[:-1]).tolist()
        d["agv_in"] = np.full(cnts[r], r, np.int16); d["agv_out"] = np.zeros(sum(cnts), np.int16); c.all_gather_v(d["agv_in"], d["agv_out"], cnts, dsp)
        d["rsv_in"] = rng.integers(0, 9, sum(cnts)).astype(np.int32); d["rsv_out"] = np.zeros(cnts[r], np.int32); c.reduce_scatter_v(d["rsv_in"], cnts, dsp, d["rsv_out"])
        d.update(cnts=cnts, dsp=dsp)
        d["sb"] = np.full(100, r, np.float32); d["rb"] = np.zeros(100, np.float32)
        if n > 1:
            hb.group_start(); c.send(d["sb"], (r + 1) % n); c.recv(d["rb"], (r - 1) % n); hb.group_end()
        c.barrier()
        out[r] = d

    run_ranks(n, body)
    for r in range(n):
        o = out[r]
        assert np.array_equal(o["y"], np.concatenate([out[q]["x"] for q in range(n)]))
        assert np.allclose(o["b"], sum(out[q]["a"][r * 777:(r + 1) * 777].astype(np.float64) for q in range(n)), atol=1e-5)
        assert np.array_equal(o["t"], np.concatenate([out[q]["s"][r * 300:(r + 1) * 300] for q in range(n)]))
        assert (o["z"] == n - 1).all()
        if r == 1 % n:
            assert np.array_equal(o["ro"], np.max([out[q]["ri"] for q in range(n)], axis=0))
        assert np.allclose(o["bo"], sum(out[q]["big"].astype(np.float64) for q in range(n)), atol=1e-5)
        assert np.array_equal(o["sc_out"], out[0]["sc_in"][r * 50:(r + 1) * 50])
        if r == n - 1:
            assert np.array_equal(o["g_out"], np.concatenate([out[q]["sc_out"] for q in range(n)]))
        assert np.array_equal(o["rv"], np.concatenate([out[q]["sv"][out[q]["sd"][r]:out[q]["sd"][r] + out[q]["sc"][r]] for q in range(n)]))
        assert np.array_equal(o["agv_out"], np.concatenate([out[q]["agv_in"] for q in range(n)]))
        assert np.array_equal(o["rsv_out"], sum(out[q]["rsv_in"][o["dsp"][r]:o["dsp"][r] + o["cnts"][r]] for q in range(n)))
        if n > 1:
            assert (o["rb"] == (r - 1) % n).all()
    destroy(comms)


def test_alltoallvc_and_batch_send_recv(monkeypatch):
    sim_env(monkeypatch)
    n = 4
    comms = make_comms(n)
    matrix = [[(i * 7 + j * 3) % 5 + 1 for j in range(n)] for i in range(n)]
    sends = [np.arange(sum(matrix[r]), dtype=np.int32) + 100 * r for r in range(n)]
    recvs = [np.zeros(sum(matrix[q][r] for q in range(n)), np.int32) for r in range(n)]
    big = [np.full(900_000, r, np.uint8) for r in range(n)]   # larger than one landing slot: several rounds
    got = [np.zeros(900_000, np.uint8) for _ in range(n)]

    def body(r):
        comms[r].all_to_all_vc(sends[r], matrix, recvs[r])
        comms[r].batch_send_recv([("send", big[r], (r + 1) % n), ("recv", got[r], (r - 1) % n)])
    run_ranks(n, body)
    for r in range(n):
        exp = []
        for q in range(n):
            off = sum(matrix[q][:r])
            exp.append(sends[q][off:off + matrix[q][r]])
        assert np.array_equal(recvs[r], np.concatenate(exp))
        assert (got[r] == (r - 1) % n).all()
    destroy(comms)


def test_sends_between_two_ranks_leave_the_collectives_of_all_ranks_intact(monkeypatch):
    """Point-to-point operators involve two ranks; the others do not count them.  Collectives before, between and after
    them must still meet in the same half of the communication buffer on every rank, and a rank that sends before it
    receives must meet a partner that has done neither yet."""
    sim_env(monkeypatch, buffsize=1)
    n = 3
    comms = make_comms(n)
    x = [np.arange(3000, dtype=np.float32) + 10 * r for r in range(n)]
    want = sum(x)
    big = np.arange(700_000, dtype=np.int32)        # larger than one landing slot: several passes
    out = [dict() for _ in range(n)]

    def body(r):
        c = comms[r]
        out[r]["a"] = c.all_reduce(x[r], np.zeros_like(x[r]))
        if r == 0:                                   # one message 0 -> 1: rank 2 knows nothing of it
            c.send(big, 1)
        elif r == 1:
            out[r]["big"] = c.recv(np.zeros_like(big), 0)
        out[r]["b"] = c.all_reduce(x[r], np.zeros_like(x[r]))
        # a ring in which ranks 0 and 2 send first and rank 1 receives first
        msg, got = np.full(100, r, np.int32), np.zeros(100, np.int32)
        if r % 2 == 0:
            c.send(msg, (r + 1) % n)
            c.recv(got, (r - 1) % n)
        else:
            c.recv(got, (r - 1) % n)
            c.send(msg, (r + 1) % n)
        out[r]["ring"] = got
        out[r]["c"] = c.all_reduce(x[r], np.zeros_like(x[r]))
        out[r]["g"] = c.all_gather(x[r], np.zeros(n * 3000, np.float32))
    run_ranks(n, body)
    for r in range(n):
        for key in "abc":
            assert np.array_equal(out[r][key], want), (r, key)
        assert np.array_equal(out[r]["g"], np.concatenate(x))
        assert (out[r]["ring"] == (r - 1) % n).all(), (r, out[r]["ring"][:4])
    assert np.array_equal(out[1]["big"], big)
    destroy(comms)


def test_sub_communicator_and_argument_checks(monkeypatch):
    sim_env(monkeypatch)
    from hcomm_b200 import HcclError
    n = 6
    comms = make_comms(n)
    evens = [0, 2, 4]
    subs = run_ranks(n, lambda r: comms[r].split(evens, sub_id=3))
    vals = [np.full(10, r + 1, np.float32) for r in range(n)]

    def body(r):
        if subs[r] is not None:
            subs[r].all_reduce(vals[r])
    run_ranks(n, body)
    for r in evens:
        assert (vals[r] == 1 + 3 + 5).all()
        assert subs[r].size == 3 and subs[r].rank == evens.index(r)
    # argument rules
    x = np.zeros(4, np.float32)
    assert comms[0].all_reduce(np.zeros(0, np.float32)) is not None          # count 0 is a successful no-op
    with pytest.raises(HcclError) as e:
        comms[0].broadcast(x, root=99)
    assert e.value.code == 1
    with pytest.raises(HcclError):
        comms[0].send(x, 0)                                                     # send to self
    run_ranks(n, lambda r: subs[r].destroy() if subs[r] else None)
    destroy(comms)


def test_rendezvous_survives_connections_that_are_not_ranks(monkeypatch):
    """Whatever connects to the rendezvous port without being a rank - silent, talking nonsense, or announcing an absurd
    message length - is dropped and does not hold up the ranks for long."""
    import socket
    import struct
    import time
    import hcomm_b200 as hb
    sim_env(monkeypatch)
    info = hb.get_root_info()
    ip = info[:64].split(b"\0")[0].decode()
    port = struct.unpack_from("<I", info, 64)[0]
    strays = []
    for payload in (None, b"GET / HTTP/1.0\r\n\r\n", struct.pack("<IHHIQQ", 0x4d434348, 1, 0, 0, 0, 1 << 60)[:24]):
        s = socket.create_connection((ip, port), timeout=5)
        if payload:
            s.sendall(payload)
        strays.append(s)            # kept open: the hub has to give up on the silent one by itself
    t0 = time.time()
    n = 3
    comms = run_ranks(n, lambda r: hb.Communicator(n, info, r))
    assert time.time() - t0 < 20
    out = run_ranks(n, lambda r: comms[r].all_reduce(np.full(100, r + 1, np.float32), np.zeros(100, np.float32)))
    assert all((o == 6).all() for o in out)
    for s in strays:
        s.close()
    destroy(comms)


def test_host_messages_between_ranks(monkeypatch):
    """Control messages over the control plane: exact and wildcard probes, order per (source, tag), an empty message."""
    import pickle
    sim_env(monkeypatch)
    n = 4
    comms = make_comms(n)
    out = [None] * n

    def body(r):
        c = comms[r]
        if r == 0:
            got = sorted(c.recv_bytes() for _ in range(2 * (n - 1)))            # from anybody, any tag
            out[r] = got
            for q in range(1, n):
                c.send_bytes(pickle.dumps({"to": q, "plan": [q] * 3}), q, tag=7)
        else:
            c.send_bytes(b"first from %d" % r, 0, tag=1)
            c.send_bytes(b"", 0, tag=2)
            assert c.probe_bytes(src=(r % (n - 1)) + 1 if (r % (n - 1)) + 1 != r else None, tag=99) is None     # nothing with that tag
            src, tag, data = c.recv_bytes(src=0, tag=7)
            out[r] = (src, tag, pickle.loads(data))
    run_ranks(n, body)
    assert out[0] == sorted([(q, 1, b"first from %d" % q) for q in range(1, n)] + [(q, 2, b"") for q in range(1, n)])
    for q in range(1, n):
        assert out[q] == (0, 7, {"to": q, "plan": [q] * 3})
    destroy(comms)


def test_configuration_values_that_make_no_sense_are_refused_at_creation(monkeypatch):
    import hcomm_b200 as hb
    sim_env(monkeypatch)
    for kw in (dict(buffer_mb=0), dict(deterministic=7), dict(op_expansion_mode=99), dict(algo="level9:zzz;;;==//"), dict(algo="level0:nosuch"),
               dict(exec_timeout=-5)):
        with pytest.raises(hb.HcclError) as err:
            hb.Communicator(1, hb.get_root_info(), 0, **kw)
        assert err.value.code == 1, kw                     # HCCL_E_PARA
    c = hb.Communicator(1, hb.get_root_info(), 0, algo="allreduce=level0:ring/others=level0:fullmesh", deterministic=1, exec_timeout=30, name="x" * 127)
    assert c.name == "x" * 127
    c.destroy()
    # the same rule for the environment variable
    monkeypatch.setenv("HCCL_ALGO", "level0:nosuch")
    from hcomm_b200 import _lib
    _lib.load().HcommToolReloadEnv()
    with pytest.raises(hb.HcclError):
        hb.Communicator(1, hb.get_root_info(), 0)
    monkeypatch.delenv("HCCL_ALGO")
    _lib.load().HcommToolReloadEnv()


@pytest.mark.parametrize("heartbeat", [False, True])
def test_communicators_destroyed_in_any_order_leave_nothing_behind(monkeypatch, heartbeat):
    """Ranks of one process, destroyed one after the other by one thread (forwards, backwards), all at once, or one first
    and the rest together: no call stalls, and descriptors and threads are back where they were."""
    import os
    import random
    import time
    import hcomm_b200 as hb
    extra = {"HCCL_HEARTBEAT_INTERVAL_MS": 50, "HCCL_HEARTBEAT_LOST_MS": 4000} if heartbeat else {}
    sim_env(monkeypatch, buffsize=1, **extra)
    rng = random.Random(5)

    def census():
        return len(os.listdir("/proc/self/fd")), len(os.listdir("/proc/self/task"))
    base = None
    t0 = time.time()
    for it in range(14):
        n = rng.choice([2, 3, 4, 5])
        info = hb.get_root_info()
        comms = run_ranks(n, lambda r: hb.Communicator(n, info, r))
        out = run_ranks(n, lambda r: comms[r].all_reduce(np.full(10, r + 1, np.float32), np.zeros(10, np.float32)))
        assert all((o == n * (n + 1) / 2).all() for o in out)
        mode = ("forwards", "backwards", "together", "one_first")[it % 4]
        if mode == "forwards":
            for c in comms:
                c.destroy()
        elif mode == "backwards":
            for c in reversed(comms):
                c.destroy()
        elif mode == "together":
            run_ranks(n, lambda r: comms[r].destroy())
        else:
            comms[0].destroy()
            run_ranks(n - 1, lambda r: comms[r + 1].destroy())
        if it == 3:
            time.sleep(0.3)
            base = census()
    time.sleep(0.3)
    assert time.time() - t0 < 60
    fds, threads = census()
    assert fds <= base[0] + 2 and threads <= base[1] + 2, (base, (fds, threads))
