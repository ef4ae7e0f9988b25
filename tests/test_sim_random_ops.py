"""Randomised operators on the host simulator against numpy: rank counts that are not powers of two, counts from zero to
several passes of the communication buffer, every forced algorithm family, roots, reductions and types drawn at random.
Integer-valued data, so that every reduction order gives the same bits."""
import os
import zlib

import numpy as np
import pytest

from helpers import run_ranks
from simutil import destroy, make_comms, sim_env

DTYPES = [np.float32, np.float64, np.int32, np.int64, np.int8, np.float16, np.uint8]
ALGOS = ["", "level0:ring", "level0:H-D_R", "level0:NHR", "level0:NB", "level0:pairwise", "level0:fullmesh"]


def _count(rng):
    kind = rng.integers(0, 6)
    if kind == 0:
        return int(rng.integers(0, 4))                    # 0, 1, 2, 3 elements
    if kind == 1:
        return int(rng.integers(4, 300))
    if kind == 2:
        return int(rng.choice([255, 256, 257, 4095, 4096, 4097, 65536 + 1]))
    if kind == 3:
        return int(rng.integers(100_000, 400_000))        # more than one pass of a 1 MB buffer for the wider types
    return int(rng.integers(300, 20_000))


def _data(rng, count, dtype, lo=-3, hi=4):
    if dtype == np.uint8:
        lo, hi = 0, 3
    return rng.integers(lo, hi, count).astype(dtype)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("n", [2, 3, 5, 6])
def test_random_operators_match_numpy(monkeypatch, algo, n):
    sim_env(monkeypatch, buffsize=1, HCCL_ALGO=algo)
    comms = make_comms(n)
    # the same draws in every run; HCOMM_TEST_SEED explores others
    rng = np.random.default_rng(zlib.crc32(f"{algo}/{n}/{os.environ.get('HCOMM_TEST_SEED', '0')}".encode()))
    for step in range(14):
        op = str(rng.choice(["all_reduce", "all_gather", "reduce_scatter", "broadcast", "reduce", "all_to_all", "scatter", "gather",
                             "all_gather_v", "reduce_scatter_v", "send_recv"]))
        dtype = DTYPES[int(rng.integers(0, len(DTYPES)))]
        count = _count(rng)
        root = int(rng.integers(0, n))
        red = str(rng.choice(["sum", "max", "min", "prod"]))
        fn = {"sum": np.sum, "max": np.max, "min": np.min, "prod": np.prod}[red]
        what = (algo, n, step, op, np.dtype(dtype).name, count, root, red)
        if red == "prod":
            lo, hi = (1, 3) if dtype != np.uint8 else (1, 2)      # products stay small
        else:
            lo, hi = -3, 4
        seeds = [int(rng.integers(0, 1 << 30)) for _ in range(n)]
        if op == "all_reduce":
            xs = [_data(np.random.default_rng(s), count, dtype, lo, hi) for s in seeds]
            in_place = bool(rng.integers(0, 2))
            outs = [x.copy() if in_place else np.zeros_like(x) for x in xs]
            run_ranks(n, lambda r: comms[r].all_reduce(outs[r] if in_place else xs[r], None if in_place else outs[r], op=red))
            ref = fn(np.stack(xs), axis=0).astype(dtype) if count else np.zeros(0, dtype)
            for r in range(n):
                assert np.array_equal(outs[r], ref), what
        elif op == "all_gather":
            xs = [_data(np.random.default_rng(s), count, dtype) for s in seeds]
            outs = [np.zeros(count * n, dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].all_gather(xs[r], outs[r]))
            for r in range(n):
                assert np.array_equal(outs[r], np.concatenate(xs)), what
        elif op == "reduce_scatter":
            xs = [_data(np.random.default_rng(s), count * n, dtype, lo, hi) for s in seeds]
            outs = [np.zeros(count, dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].reduce_scatter(xs[r], outs[r], op=red))
            ref = fn(np.stack(xs), axis=0).astype(dtype) if count else np.zeros(0, dtype)
            for r in range(n):
                assert np.array_equal(outs[r], ref[r * count:(r + 1) * count]), what
        elif op == "broadcast":
            xs = [_data(np.random.default_rng(s), count, dtype) for s in seeds]
            bufs = [x.copy() for x in xs]
            run_ranks(n, lambda r: comms[r].broadcast(bufs[r], root=root))
            for r in range(n):
                assert np.array_equal(bufs[r], xs[root]), what
        elif op == "reduce":
            xs = [_data(np.random.default_rng(s), count, dtype, lo, hi) for s in seeds]
            outs = [np.zeros_like(x) for x in xs]
            run_ranks(n, lambda r: comms[r].reduce(xs[r], outs[r], root=root, op=red))
            ref = fn(np.stack(xs), axis=0).astype(dtype) if count else np.zeros(0, dtype)
            assert np.array_equal(outs[root], ref), what
        elif op == "all_to_all":
            count = min(count, 60_000)
            xs = [_data(np.random.default_rng(s), count * n, dtype) for s in seeds]
            outs = [np.zeros(count * n, dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].all_to_all(xs[r], outs[r]))
            for r in range(n):
                ref = np.concatenate([xs[q][r * count:(r + 1) * count] for q in range(n)]) if count else np.zeros(0, dtype)
                assert np.array_equal(outs[r], ref), what
        elif op == "scatter":
            count = min(count, 100_000)
            xs = [_data(np.random.default_rng(s), count * n, dtype) for s in seeds]
            outs = [np.zeros(count, dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].scatter(xs[r], outs[r], root=root))
            for r in range(n):
                assert np.array_equal(outs[r], xs[root][r * count:(r + 1) * count]), what
        elif op == "gather":
            count = min(count, 100_000)
            xs = [_data(np.random.default_rng(s), count, dtype) for s in seeds]
            outs = [np.zeros(count * n, dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].gather(xs[r], outs[r], root=root))
            assert np.array_equal(outs[root], np.concatenate(xs)), what
        elif op == "all_gather_v":
            counts = [int(c) for c in rng.integers(0, max(2, min(count, 50_000)), n)]
            displs = [int(d) for d in np.concatenate([[0], np.cumsum(counts)[:-1]])]
            xs = [_data(np.random.default_rng(seeds[r]), counts[r], dtype) for r in range(n)]
            outs = [np.zeros(sum(counts), dtype) for _ in range(n)]
            run_ranks(n, lambda r: comms[r].all_gather_v(xs[r], outs[r], counts, displs))
            for r in range(n):
                assert np.array_equal(outs[r], np.concatenate(xs)), what + (counts,)
        elif op == "reduce_scatter_v":
            counts = [int(c) for c in rng.integers(0, max(2, min(count, 50_000)), n)]
            displs = [int(d) for d in np.concatenate([[0], np.cumsum(counts)[:-1]])]
            xs = [_data(np.random.default_rng(s), sum(counts), dtype, lo, hi) for s in seeds]
            outs = [np.zeros(counts[r], dtype) for r in range(n)]
            run_ranks(n, lambda r: comms[r].reduce_scatter_v(xs[r], counts, displs, outs[r], op=red))
            ref = fn(np.stack(xs), axis=0).astype(dtype) if sum(counts) else np.zeros(0, dtype)
            for r in range(n):
                assert np.array_equal(outs[r], ref[displs[r]:displs[r] + counts[r]]), what + (counts,)
        elif op == "send_recv":
            # a few messages between random pairs; ranks that are not named do nothing
            src, dst = (int(v) for v in rng.choice(n, 2, replace=False))
            msg = _data(np.random.default_rng(seeds[0]), count, dtype)
            got = np.zeros(count, dtype)

            def body(r):
                if r == src:
                    comms[r].send(msg, dst)
                elif r == dst:
                    comms[r].recv(got, src)
            run_ranks(n, body)
            assert np.array_equal(got, msg), what
    destroy(comms)
