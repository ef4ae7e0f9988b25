"""The SM-engine collective kernels, several ranks sharing one GPU in one cooperative launch,
checked against plain PyTorch fp32 (or exact integer) references."""
import os

import pytest
import torch

from helpers import run_ranks

pytestmark = pytest.mark.gpu


def _make(n, **kw):
    import hcomm_b200 as hb
    info = hb.get_root_info()

    def init(r):
        torch.cuda.set_device(0)
        return hb.Communicator(n, info, r, buffer_mb=kw.get("buffer_mb", 8), **{k: v for k, v in kw.items() if k != "buffer_mb"})
    return run_ranks(n, init)


def _destroy(comms):
    run_ranks(len(comms), lambda r: comms[r].destroy())


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32])
def test_allreduce_small_and_large(n, dtype):
    comms = _make(n)
    try:
        for count in (1, 7, 1000, 65536, 1_000_003):
            gen = torch.Generator(device="cuda").manual_seed(count)
            if dtype.is_floating_point:
                xs = [torch.randn(count, device="cuda", generator=gen).to(dtype) for _ in range(n)]
            else:
                xs = [torch.randint(-1000, 1000, (count,), device="cuda", generator=gen, dtype=dtype) for _ in range(n)]
            outs = [torch.empty_like(x) for x in xs]

            def op(r):
                torch.cuda.set_device(0)
                comms[r].all_reduce(xs[r], outs[r])
                torch.cuda.synchronize()
            run_ranks(n, op)
            ref = sum(x.double() for x in xs)
            for r in range(n):
                assert torch.equal(outs[r], outs[0]), "ranks disagree"
            if dtype.is_floating_point:
                tol = {torch.float32: 1e-5, torch.bfloat16: 4e-2, torch.float16: 4e-3}[dtype] * (n ** 0.5) * 4
                assert (outs[0].double() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
            else:
                assert torch.equal(outs[0].double(), ref)
    finally:
        _destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 8])
def test_reduce_scatter_allgather_alltoall_broadcast(n):
    comms = _make(n)
    try:
        per = 4099
        xs = [torch.randn(per * n, device="cuda") for _ in range(n)]
        rs = [torch.empty(per, device="cuda") for _ in range(n)]
        ag_in = [torch.randn(per, device="cuda").to(torch.bfloat16) for _ in range(n)]
        ag_out = [torch.empty(per * n, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        a2a_in = [torch.arange(per * n, device="cuda", dtype=torch.int32) + 1_000_000 * r for r in range(n)]
        a2a_out = [torch.empty(per * n, device="cuda", dtype=torch.int32) for _ in range(n)]
        bc = [torch.full((123457,), float(r), device="cuda") for r in range(n)]
        red_out = [torch.empty(per * n, device="cuda") for _ in range(n)]

        def op(r):
            torch.cuda.set_device(0)
            c = comms[r]
            c.reduce_scatter(xs[r], rs[r])
            c.all_gather(ag_in[r], ag_out[r])
            c.all_to_all(a2a_in[r], a2a_out[r])
            c.broadcast(bc[r], root=n - 1)
            c.reduce(xs[r], red_out[r], root=0, op="max")
            c.barrier()
            torch.cuda.synchronize()
        run_ranks(n, op)
        total = sum(x.double() for x in xs)
        for r in range(n):
            assert (rs[r].double() - total[r * per:(r + 1) * per]).abs().max().item() < 1e-4
            assert torch.equal(ag_out[r], torch.cat(ag_in))
            assert torch.equal(a2a_out[r], torch.cat([a2a_in[q][r * per:(r + 1) * per] for q in range(n)]))
            assert (bc[r] == n - 1).all()
        assert torch.equal(red_out[0], torch.stack(xs).max(dim=0).values)
    finally:
        _destroy(comms)


def test_chunked_allreduce_and_scaled(n=4):
    comms = _make(n, buffer_mb=1)     # 1 MB halves force several launches per operator
    try:
        count = 3_000_001
        xs = [torch.randn(count, device="cuda").to(torch.bfloat16) for _ in range(n)]
        outs = [torch.empty_like(x) for x in xs]

        def op(r):
            torch.cuda.set_device(0)
            comms[r].all_reduce_scaled(xs[r], outs[r], scale=1.0 / n)
            torch.cuda.synchronize()
        run_ranks(n, op)
        ref = sum(x.float() for x in xs) / n
        assert torch.equal(outs[1], outs[0])
        assert (outs[0].float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    finally:
        _destroy(comms)


def test_alltoallv_variable_counts(n=4):
    comms = _make(n)
    try:
        sc = [[(r * 3 + q * 5) % 7 * 1000 + 17 for q in range(n)] for r in range(n)]
        rc = [[sc[q][r] for q in range(n)] for r in range(n)]
        sd = [[sum(sc[r][:q]) for q in range(n)] for r in range(n)]
        rd = [[sum(rc[r][:q]) for q in range(n)] for r in range(n)]
        send = [torch.arange(sum(sc[r]), device="cuda", dtype=torch.float32) + 1e6 * r for r in range(n)]
        recv = [torch.empty(sum(rc[r]), device="cuda") for r in range(n)]

        def op(r):
            torch.cuda.set_device(0)
            comms[r].all_to_all_v(send[r], sc[r], sd[r], recv[r], rc[r], rd[r])
            torch.cuda.synchronize()
        run_ranks(n, op)
        for r in range(n):
            exp = torch.cat([send[q][sd[q][r]:sd[q][r] + sc[q][r]] for q in range(n)])
            assert torch.equal(recv[r], exp)
    finally:
        _destroy(comms)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_small_message_flag_in_data_kernel(n):
    """Blocks that are whole 16-byte vectors of at most 32 KB take the barrier-free kernel: repeated calls (the tag and
    the slot parity advance), in-place all-reduce, and large operators in between."""
    comms = _make(n)
    try:
        per = 2048                                   # 8 KB fp32 blocks
        for rep in range(5):
            g = torch.Generator(device="cuda").manual_seed(100 + rep)
            xs = [torch.randn(per * n, device="cuda", generator=g) for _ in range(n)]
            ar = [x[:per].clone() for x in xs]
            rs = [torch.empty(per, device="cuda") for _ in range(n)]
            ag_out = [torch.empty(per * n, device="cuda") for _ in range(n)]
            a2a_out = [torch.empty(per * n, device="cuda") for _ in range(n)]
            big = [torch.randn(300_000, device="cuda", generator=g) for _ in range(n)]
            big_out = [torch.empty_like(b) for b in big]
            half = [x[:per].to(torch.bfloat16) for x in xs]
            half_out = [torch.empty_like(h) for h in half]

            def op(r):
                torch.cuda.set_device(0)
                c = comms[r]
                c.all_reduce(ar[r])                              # in place
                c.reduce_scatter(xs[r], rs[r])
                c.all_gather(xs[r][:per], ag_out[r])
                if rep % 2:
                    c.all_reduce(big[r], big_out[r])             # a barrier-based kernel between the small ones
                c.all_to_all(xs[r], a2a_out[r])
                c.all_reduce(half[r], half_out[r], op="max")
                torch.cuda.synchronize()
            run_ranks(n, op)
            total = sum(x.double() for x in xs)
            for r in range(n):
                assert torch.equal(ar[r], ar[0])
                assert (ar[r].double() - total[:per]).abs().max().item() < 1e-4
                assert (rs[r].double() - total[r * per:(r + 1) * per]).abs().max().item() < 1e-4
                assert torch.equal(ag_out[r], torch.cat([x[:per] for x in xs]))
                assert torch.equal(a2a_out[r], torch.cat([xs[q][r * per:(r + 1) * per] for q in range(n)]))
                assert torch.equal(half_out[r], torch.stack(half).max(dim=0).values)
            assert all(c.async_error() == 0 for c in comms)
    finally:
        _destroy(comms)


@pytest.mark.parametrize("n,algo", [(2, "level0:ring"), (4, "level0:ring"), (4, "level0:H-D_R"), (3, "level0:H-D_R"), (4, "level0:pairwise"), (8, "level0:NB"),
                                    (8, "level0:ring")])
def test_forced_algorithms_run_in_the_schedule_interpreter(n, algo):
    """Ring, halving-doubling (with a non-power-of-two fold), pairwise and Bruck schedules, executed by the interpreter
    kernel; a 1 MB buffer forces several column passes for the larger vectors."""
    comms = _make(n, buffer_mb=1, algo=algo)
    try:
        for count in (1000, 70_001, 1_200_007):
            g = torch.Generator(device="cuda").manual_seed(count)
            xs = [torch.randn(count, device="cuda", generator=g) for _ in range(n)]
            outs = [torch.empty_like(x) for x in xs]
            per = max(1, count // n)
            ag_in = [torch.randint(0, 1 << 20, (per,), device="cuda", generator=g, dtype=torch.int32) for _ in range(n)]
            ag_out = [torch.empty(per * n, device="cuda", dtype=torch.int32) for _ in range(n)]
            rs_in = [torch.randn(per * n, device="cuda", generator=g).to(torch.bfloat16) for _ in range(n)]
            rs_out = [torch.empty(per, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
            a2a_in = [torch.arange(per * n, device="cuda", dtype=torch.int32) + 10_000_000 * r for r in range(n)]
            a2a_out = [torch.empty(per * n, device="cuda", dtype=torch.int32) for _ in range(n)]
            bc = [torch.full((count,), float(r), device="cuda") for r in range(n)]

            def op(r):
                torch.cuda.set_device(0)
                c = comms[r]
                c.all_reduce(xs[r], outs[r])
                c.all_gather(ag_in[r], ag_out[r])
                c.reduce_scatter(rs_in[r], rs_out[r])
                c.all_to_all(a2a_in[r], a2a_out[r])
                c.broadcast(bc[r], root=1)
                torch.cuda.synchronize()
            run_ranks(n, op)
            ref = sum(x.double() for x in xs)
            total = sum(x.double() for x in rs_in)
            for r in range(n):
                assert (outs[r].double() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item()), (algo, count, "all_reduce")
                assert torch.equal(ag_out[r], torch.cat(ag_in)), (algo, count, "all_gather")
                assert (rs_out[r].double() - total[r * per:(r + 1) * per]).abs().max().item() <= 0.1 * (n ** 0.5), (algo, count, "reduce_scatter")
                assert torch.equal(a2a_out[r], torch.cat([a2a_in[q][r * per:(r + 1) * per] for q in range(n)])), (algo, count, "all_to_all")
                assert (bc[r] == 1).all(), (algo, count, "broadcast")
            assert all(c.async_error() == 0 for c in comms)
    finally:
        _destroy(comms)


@pytest.mark.parametrize("n", [2, 4])
def test_buffers_that_are_not_16_byte_aligned(n):
    """Views that start one element into an allocation: the operators must not depend on vector alignment."""
    comms = _make(n)
    try:
        for dtype, count in ((torch.bfloat16, 300_001), (torch.float32, 70_003)):
            g = torch.Generator(device="cuda").manual_seed(count)
            base_in = [torch.randn(count * n + 8, device="cuda", generator=g).to(dtype) for _ in range(n)]
            base_out = [torch.zeros(count * n + 8, device="cuda", dtype=dtype) for _ in range(n)]
            xs = [b[1:1 + count] for b in base_in]
            outs = [b[3:3 + count] for b in base_out]
            ag_out = [torch.zeros(count * n + 8, device="cuda", dtype=dtype) for _ in range(n)]
            rs_in = [b[1:1 + count * n] for b in base_in]
            rs_out = [torch.zeros(count + 8, device="cuda", dtype=dtype) for _ in range(n)]

            def op(r):
                torch.cuda.set_device(0)
                comms[r].all_reduce(xs[r], outs[r])
                comms[r].all_gather(xs[r], ag_out[r][1:1 + count * n])
                comms[r].reduce_scatter(rs_in[r], rs_out[r][1:1 + count])
                torch.cuda.synchronize()
            run_ranks(n, op)
            ref = sum(x.double() for x in xs)
            total = sum(x.double() for x in rs_in)
            tol = (1e-5 if dtype == torch.float32 else 4e-2) * (n ** 0.5) * 4
            for r in range(n):
                assert (outs[r].double() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
                assert torch.equal(ag_out[r][1:1 + count * n], torch.cat(xs))
                assert (rs_out[r][1:1 + count].double() - total[r * count:(r + 1) * count]).abs().max().item() <= tol * max(1.0, total.abs().max().item())
                assert base_out[r][0] == 0 and base_out[r][3 + count] == 0 and ag_out[r][0] == 0      # nothing outside the views was touched
            assert all(c.async_error() == 0 for c in comms)
    finally:
        _destroy(comms)


@pytest.mark.parametrize("n", [2, 4])
def test_blocks_at_displacements_that_are_not_16_byte_aligned(n):
    """Aligned buffers whose per-rank blocks have an odd length: one phase of the specialised kernels can use vector
    accesses and the other cannot, and both must still give the same bytes to the same CTA.  Repeated, with a small
    staging buffer (several windows) and with the default one, because a wrong split shows as a race."""
    for buffer_mb in (1, 64):
        comms = _make(n, buffer_mb=buffer_mb)
        try:
            for dtype, per in ((torch.int32, 600_003), (torch.bfloat16, 300_001), (torch.int32, 70_001)):
                ag_in = [(torch.arange(per, device="cuda", dtype=torch.int32) + 1_000_000 * r).to(dtype) for r in range(n)]
                a2a_in = [(torch.arange(per * n, device="cuda", dtype=torch.int32) + 10_000_000 * r).to(dtype) for r in range(n)]
                rs_in = [((torch.arange(per * n, device="cuda", dtype=torch.int32) + r) % 64).to(dtype) for r in range(n)]
                for rep in range(4):
                    ag_out = [torch.zeros(per * n, device="cuda", dtype=dtype) for _ in range(n)]
                    a2a_out = [torch.zeros(per * n, device="cuda", dtype=dtype) for _ in range(n)]
                    rs_out = [torch.zeros(per, device="cuda", dtype=dtype) for _ in range(n)]

                    def op(r):
                        torch.cuda.set_device(0)
                        comms[r].all_gather(ag_in[r], ag_out[r])
                        comms[r].all_to_all(a2a_in[r], a2a_out[r])
                        comms[r].reduce_scatter(rs_in[r], rs_out[r])
                        torch.cuda.synchronize()
                    run_ranks(n, op)
                    total = sum(x.double() for x in rs_in)     # sums of small integers: exact in bf16 too
                    for r in range(n):
                        assert torch.equal(ag_out[r], torch.cat(ag_in)), (buffer_mb, dtype, per, rep, "all_gather")
                        assert torch.equal(a2a_out[r], torch.cat([a2a_in[q][r * per:(r + 1) * per] for q in range(n)])), (buffer_mb, dtype, per, rep, "all_to_all")
                        assert torch.equal(rs_out[r].double(), total[r * per:(r + 1) * per]), (buffer_mb, dtype, per, rep, "reduce_scatter")
            assert all(c.async_error() == 0 for c in comms)
        finally:
            _destroy(comms)


def test_kernel_time_ring_reports_device_durations(n=2):
    comms = _make(n)
    try:
        xs = [torch.randn(1 << 20, device="cuda") for _ in range(n)]
        outs = [torch.empty_like(x) for x in xs]

        def op(r):
            torch.cuda.set_device(0)
            comms[r].all_reduce(xs[r], outs[r])                      # before profiling is switched on: not recorded
            torch.cuda.synchronize()
            comms[r].set_profiling(True)
            for _ in range(5):
                comms[r].all_reduce(xs[r], outs[r])
            torch.cuda.synchronize()
        run_ranks(n, op)
        times = comms[0].kernel_times()
        assert len(times) == 5
        for start, end in times:
            assert start > 0 and end >= start and end - start < 1_000_000_000
        assert all(times[i][0] <= times[i + 1][0] for i in range(len(times) - 1))
        assert "allreduce" in comms[0].dump().lower().replace("_", "")
    finally:
        _destroy(comms)


def test_single_rank_operator_in_a_captured_cuda_graph():
    """The demo of examples/02_graphs on one GPU (one rank): capture, replay with new data."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    res = subprocess.run([sys.executable, str(root / "examples" / "02_graphs" / "allreduce_cuda_graph_demo.py")], capture_output=True, text=True, timeout=240)
    assert res.returncode == 0 and "5 replays ok" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
