"""Helpers for tests that run ranks as threads on the host simulator."""
import ctypes
import os

import numpy as np

from helpers import run_ranks

CMD = dict(broadcast=1, allreduce=2, reduce=3, send=4, receive=5, allgather=6, reducescatter=7, alltoallv=8, alltoallvc=9, alltoall=10, gather=11,
           scatter=12)


def sim_env(monkeypatch, **extra):
    monkeypatch.setenv("HCCL_SIM", "1")
    monkeypatch.setenv("HCCL_BUFFSIZE", str(extra.pop("buffsize", 2)))
    for k, v in extra.items():
        monkeypatch.setenv(k, str(v))
    from hcomm_b200 import _lib
    _lib.load().HcommToolReloadEnv()


def make_comms(n, **kw):
    import hcomm_b200 as hb
    info = hb.get_root_info()
    return run_ranks(n, lambda r: hb.Communicator(n, info, r, **kw))


def destroy(comms):
    run_ranks(len(comms), lambda r: comms[r].destroy())


def tool_str(fn, *args, size=1 << 16):
    buf = ctypes.create_string_buffer(size)
    rc = fn(*args, buf, size)
    return rc, buf.value.decode(errors="replace")
