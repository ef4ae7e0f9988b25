"""One rank of a multi-process test; started by test_multigpu.py / test_multiprocess_sim.py.

argv: scenario name.  Environment: RANK, WORLD_SIZE, LOCAL_RANK, HCOMM_ROOT_FILE (rank 0 writes the
rendezvous ticket there, the others poll for it).
"""
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import numpy as np  # noqa: E402


def root_info(rank):
    import hcomm_b200 as hb
    path = Path(os.environ["HCOMM_ROOT_FILE"])
    if rank == 0:
        info = hb.get_root_info()
        tmp = path.with_suffix(".tmp")
        tmp.write_bytes(info)
        tmp.rename(path)
        return info
    deadline = time.time() + 60
    while not path.exists():
        if time.time() > deadline:
            raise TimeoutError("no root info file")
        time.sleep(0.02)
    return path.read_bytes()


def torch_scenario(scenario, rank, world, local, use_cuda):
    """torch.distributed over the "hccl" backend: every c10d operator against values computable locally."""
    import torch
    import torch.distributed as dist
    import hcomm_b200.parallel.backend  # noqa: F401  (registers the backend)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("hccl", rank=rank, world_size=world)

    def val(r, n, dtype=torch.float32):
        return (torch.arange(n, dtype=torch.float32) * 0.25 + r + 1).to(dtype).to(dev)

    if scenario == "torch_ops":
        n = 1000
        t = val(rank, n)
        dist.all_reduce(t)
        want = sum(val(r, n) for r in range(world))
        assert torch.allclose(t, want), "all_reduce"
        t = val(rank, n)
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        assert torch.allclose(t, want / world, rtol=1e-5), "all_reduce avg"
        t = val(rank, n)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert torch.equal(t, val(world - 1, n)), "all_reduce max"
        t = val(rank, n, torch.int64)
        dist.all_reduce(t)
        assert torch.equal(t, sum(val(r, n, torch.int64) for r in range(world))), "all_reduce int64"
        t = val(rank, n)
        dist.broadcast(t, src=1)
        assert torch.equal(t, val(1, n)), "broadcast"
        outs = [torch.empty(n, device=dev) for _ in range(world)]
        dist.all_gather(outs, val(rank, n))
        assert all(torch.equal(outs[r], val(r, n)) for r in range(world)), "all_gather"
        flat = torch.empty(world * n, device=dev)
        dist.all_gather_into_tensor(flat, val(rank, n))
        assert torch.equal(flat, torch.cat([val(r, n) for r in range(world)])), "all_gather_into_tensor"
        out = torch.empty(n, device=dev)
        dist.reduce_scatter_tensor(out, torch.cat([val(rank, n) * (q + 1) for q in range(world)]))
        assert torch.allclose(out, want * (rank + 1)), "reduce_scatter_tensor"
        out = torch.empty(n, device=dev)
        dist.reduce_scatter(out, [val(rank, n) * (q + 1) for q in range(world)])
        assert torch.allclose(out, want * (rank + 1)), "reduce_scatter"
        t = val(rank, n)
        dist.reduce(t, dst=0)
        if rank == 0:
            assert torch.allclose(t, want), "reduce"
        send = torch.cat([val(rank, 8) + 100 * q for q in range(world)])
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        assert torch.equal(recv, torch.cat([val(q, 8) + 100 * rank for q in range(world)])), "all_to_all_single"
        # uneven splits: rank r sends (q + 1) rows of 4 to rank q
        rows_out = [q + 1 for q in range(world)]
        rows_in = [rank + 1] * world
        send = torch.cat([torch.full((q + 1, 4), float(10 * rank + q), device=dev) for q in range(world)])
        recv = torch.empty(sum(rows_in), 4, device=dev)
        dist.all_to_all_single(recv, send, output_split_sizes=rows_in, input_split_sizes=rows_out)
        assert torch.equal(recv, torch.cat([torch.full((rank + 1, 4), float(10 * q + rank), device=dev) for q in range(world)])), "all_to_all_single splits"
        outs = [torch.empty(q + 2, device=dev) for q in range(world)]
        outs = [torch.empty(rank + 2, device=dev) for _ in range(world)]
        dist.all_to_all(outs, [torch.full((q + 2,), float(rank), device=dev) for q in range(world)])
        assert all(torch.equal(outs[q], torch.full((rank + 2,), float(q), device=dev)) for q in range(world)), "all_to_all"
        gl = [torch.empty(n, device=dev) for _ in range(world)] if rank == 0 else None
        dist.gather(val(rank, n), gl, dst=0)
        if rank == 0:
            assert all(torch.equal(gl[r], val(r, n)) for r in range(world)), "gather"
        out = torch.empty(n, device=dev)
        dist.scatter(out, [val(q, n) * 3 for q in range(world)] if rank == 0 else None, src=0)
        assert torch.equal(out, val(rank, n) * 3), "scatter"
        if world >= 2:
            if rank == 0:
                dist.send(val(7, n), dst=1)
            elif rank == 1:
                t = torch.empty(n, device=dev)
                dist.recv(t, src=0)
                assert torch.equal(t, val(7, n)), "send/recv"
        dist.barrier()
        work = dist.all_reduce(val(rank, n), async_op=True)
        work.wait()
        assert work.is_completed() or use_cuda
        print(f"rank {rank}: torch operators ok", flush=True)
    elif scenario == "torch_ddp":
        from hcomm_b200.parallel.ddp import wrap
        torch.manual_seed(1234)
        dtype = torch.bfloat16 if use_cuda else torch.float32
        net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).to(dev).to(dtype)
        ref = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).to(dev).to(dtype)
        ref.load_state_dict(net.state_dict())
        ddp = wrap(net, bucket_cap_mb=1)
        g = torch.Generator().manual_seed(99)
        xs = torch.randn(world, 16, 64, generator=g).to(dtype)
        ys = torch.randn(world, 16, 32, generator=g).to(dtype)
        opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
        ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
        for step in range(3):
            opt.zero_grad(set_to_none=True)
            loss = torch.nn.functional.mse_loss(ddp(xs[rank].to(dev)).float(), ys[rank].to(dev).float())
            loss.backward()
            opt.step()
            # reference: the mean over ranks of the per-rank gradients, computed locally
            ropt.zero_grad(set_to_none=True)
            total = sum(torch.nn.functional.mse_loss(ref(xs[r].to(dev)).float(), ys[r].to(dev).float()) for r in range(world)) / world
            total.backward()
            ropt.step()
        tol = 3e-2 if use_cuda else 1e-5
        for a, b in zip(net.parameters(), ref.parameters()):
            assert torch.allclose(a.float(), b.float(), rtol=tol, atol=tol), (step, (a.float() - b.float()).abs().max().item())
        print(f"rank {rank}: ddp ok", flush=True)
    if use_cuda:
        torch.cuda.synchronize()
    dist.destroy_process_group()
    return 0


def main():
    scenario = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    import hcomm_b200 as hb
    use_cuda = os.environ.get("HCCL_SIM") != "1"
    if use_cuda:
        import torch
        torch.cuda.set_device(local)

    if scenario == "never_join" and rank == world - 1:
        return 0   # this rank never joins the rendezvous
    if scenario.startswith("torch_"):
        return torch_scenario(scenario, rank, world, local, use_cuda)
    if scenario == "hcom_master_info":
        # Nobody is given a rank: every process knows the master's address only.  The process that gets the port serves.
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()
        port = os.environ["HCOMM_TEST_MASTER_PORT"].encode()
        assert lib.HcomInitByMasterInfo(b"127.0.0.1", b"notaport", b"0", str(world).encode(), b"127.0.0.1") == 1
        rc = lib.HcomInitByMasterInfo(b"127.0.0.1", port, b"0", str(world).encode(), b"127.0.0.1")
        assert rc == 0, rc
        size, me = ctypes.c_uint32(), ctypes.c_uint32()
        assert lib.HcomGetRankSize(b"hccl_world_group", ctypes.byref(size)) == 0 and size.value == world
        assert lib.HcomGetRankId(b"hccl_world_group", ctypes.byref(me)) == 0 and me.value < world
        x = np.zeros(world, np.float32)
        x[me.value] = 1.0                                  # every rank marks its own slot: the ranks handed out are all different
        y = np.zeros_like(x)
        V = ctypes.c_void_p
        assert lib.HcomAllReduce(b"t", x.ctypes.data_as(V), y.ctypes.data_as(V), ctypes.c_uint64(world), 4, 0, b"hccl_world_group", None) == 0
        assert (y == 1).all(), y
        assert lib.HcomInitByMasterInfo(b"127.0.0.1", port, b"0", str(world).encode(), b"127.0.0.1") == 1      # already there
        assert lib.HcomDestroy() == 0
        print(f"process {rank}: was rank {me.value}, ok", flush=True)
        return 0
    kw = {}
    if os.environ.get("HCOMM_TEST_BUFFER_MB"):
        kw["buffer_mb"] = int(os.environ["HCOMM_TEST_BUFFER_MB"])
    try:
        comm = hb.Communicator(world, root_info(rank), rank, **kw)
    except hb.HcclError as e:
        print(f"rank {rank}: init failed with {e.code}", flush=True)
        return 40 + e.code

    def stage(msg):
        print(f"rank {rank}: {msg}", flush=True)

    stage("communicator ready")
    if scenario in ("collectives", "never_join"):
        if use_cuda:
            import torch
            for dtype in (torch.float32, torch.bfloat16):
                for count in (1, 1024, 1 << 20, 5_000_011):
                    x = (torch.arange(count, device="cuda", dtype=torch.float32) % 13 + rank).to(dtype)
                    y = torch.empty_like(x)
                    comm.all_reduce(x, y)
                    ref = sum((torch.arange(count, device="cuda", dtype=torch.float32) % 13 + r) for r in range(world))
                    torch.cuda.synchronize()
                    assert torch.allclose(y.float(), ref.to(dtype).float(), rtol=2e-2, atol=1e-3), (dtype, count)
                    assert comm.async_error() == 0, f"async error after all_reduce {dtype} {count}"
                    stage(f"all_reduce {dtype} {count} ok")
            per = 70001
            xi = torch.full((per,), float(rank), device="cuda")
            yo = torch.empty(per * world, device="cuda")
            comm.all_gather(xi, yo)
            torch.cuda.synchronize(); stage("all_gather done")
            a2a_in = torch.arange(per * world, device="cuda", dtype=torch.int32) + 1_000_000 * rank
            a2a_out = torch.empty_like(a2a_in)
            comm.all_to_all(a2a_in, a2a_out)
            rs_out = torch.empty(per, device="cuda")
            comm.reduce_scatter(yo, rs_out)
            b = torch.full((300_001,), float(rank), device="cuda")
            comm.broadcast(b, root=world - 1)
            torch.cuda.synchronize(); stage("all_to_all, reduce_scatter, broadcast done")
            # ring exchange with the send/recv kernels
            sb, rb = torch.full((3_000_000,), float(rank), device="cuda"), torch.empty(3_000_000, device="cuda")
            hb.group_start(); comm.send(sb, (rank + 1) % world); comm.recv(rb, (rank - 1) % world); hb.group_end()
            torch.cuda.synchronize(); stage("send/recv done")
            comm.barrier()
            torch.cuda.synchronize()
            assert torch.equal(yo, torch.arange(world, device="cuda").repeat_interleave(per).float())
            assert torch.equal(a2a_out, torch.cat([torch.arange(rank * per, (rank + 1) * per, device="cuda", dtype=torch.int32) + 1_000_000 * q for q in range(world)]))
            assert torch.equal(rs_out, torch.full((per,), float(rank * world), device="cuda"))
            assert (b == world - 1).all()
            assert (rb == (rank - 1) % world).all()
            assert comm.async_error() == 0
        else:
            x = np.full(100_000, rank + 1, np.float32)
            y = np.zeros_like(x)
            comm.all_reduce(x, y)
            assert (y == world * (world + 1) / 2).all()
            g = np.zeros(7 * world, np.int32)
            comm.all_gather(np.full(7, rank, np.int32), g)
            assert np.array_equal(g, np.repeat(np.arange(world), 7))
    elif scenario == "collectives_big":
        # Operands larger than the staging (in-kernel windows), the in-switch (NVLS) kernels forced with many CTAs on counts
        # that do not divide evenly, and zero-copy on registered buffers - each against values computed locally.
        import torch
        nvls_ok = world > 1 and os.environ.get("HCCL_NVLS_ENABLE", "1") != "0"

        def pattern(count, r, dtype):
            return (torch.arange(count, device="cuda", dtype=torch.float32) % 13 + r).to(dtype)

        def check_all(c, tag, dtype, count, registered=False):
            want_ar = sum(pattern(count, r, torch.float32) for r in range(world)).to(dtype).float()
            per = count // world
            if registered:
                x, y = c.alloc_registered((count,), dtype), c.alloc_registered((count,), dtype)
                x.copy_(pattern(count, rank, dtype))
            else:
                x, y = pattern(count, rank, dtype), torch.empty(count, device="cuda", dtype=dtype)
            y.zero_()
            c.all_reduce(x, y)
            torch.cuda.synchronize()
            assert torch.allclose(y.float(), want_ar, rtol=2e-2, atol=1e-3), (tag, "all_reduce", dtype, count)
            if per * world == count and per > 0:
                rs = torch.zeros(per, device="cuda", dtype=dtype)
                c.reduce_scatter(x, rs)
                torch.cuda.synchronize()
                assert torch.allclose(rs.float(), want_ar[rank * per:(rank + 1) * per], rtol=2e-2, atol=1e-3), (tag, "reduce_scatter", dtype, count)
                y.zero_()
                c.all_gather(x[:per], y)
                torch.cuda.synchronize()
                want_ag = torch.cat([pattern(count, r, dtype)[:per] for r in range(world)])
                assert torch.equal(y, want_ag), (tag, "all_gather", dtype, count)
            assert c.async_error() == 0, (tag, dtype, count)
            stage(f"{tag}: {dtype} x {count} ok")

        # 16 MB of CCL buffer: these operands take several windows per launch
        for dtype, count in ((torch.float32, 9_000_000 * world // world // world * world), (torch.bfloat16, 24 * 1024 * 1024 + 16 * world)):
            check_all(comm, "windows", dtype, count // world * world)
        check_all(comm, "ragged", torch.float32, 5_000_011)
        if nvls_ok:
            forced = comm.split(list(range(world)), sub_id=7, buffer_mb=int(os.environ.get("HCOMM_TEST_BUFFER_MB", "16")),
                                algo="allreduce=level0:nvls/allgather=level0:nvls/reducescatter=level0:nvls")
            # 144 CTAs x 512 threads = 73728 vectors per sweep; these counts leave partial sweeps on every rank
            for dtype, count in ((torch.float32, (73728 * 4 * 3 + 40) * world), (torch.bfloat16, (73728 * 8 * 2 + 4104) * world), (torch.float32, 20_000_000 // world * world),
                                 (torch.bfloat16, 40_000_000 // (8 * world) * (8 * world))):
                # the two 80 MB operands take the pipelined kernel (the test lowers its threshold to 32 MB): ten windows
                check_all(forced, "nvls forced", dtype, count)
            check_all(forced, "nvls forced, ragged", torch.bfloat16, 3_000_001)
            forced.destroy()
        for dtype, count in ((torch.float32, 1 << 20), (torch.bfloat16, (6 << 20) + 8 * world), (torch.float32, 12_000_000 // world * world)):
            check_all(comm, "registered", dtype, count, registered=True)
        stage("collectives_big ok")
    elif scenario == "fused":
        import torch
        from hcomm_b200.ops.fused import all_gather_gemm, gemm_reduce_scatter
        from hcomm_b200.ops.gemm import take_kernel_error
        from hcomm_b200.ops.moe import MoeExchange, quantize_e4m3_1x128
        import torch.distributed as dist
        dist.init_process_group("gloo", init_method=f"file://{os.environ['HCOMM_ROOT_FILE']}.gloo", rank=rank, world_size=world)
        m, n_, k = 128 * world * 2, 512, 1024
        g = torch.Generator(device="cuda").manual_seed(5 + rank)
        a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        b = (torch.randn(n_, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        for rep in range(3):
            y = gemm_reduce_scatter(comm, a, b)
            torch.cuda.synchronize()
            part = (a.float() @ b.float().t()).cpu()
            dist.all_reduce(part)
            rows = m // world
            err = (y.float().cpu() - part[rank * rows:(rank + 1) * rows]).abs().max().item()
            assert err <= 2e-2 * max(1.0, part.abs().max().item()), ("gemm_rs", rep, err)
        stage("gemm_reduce_scatter ok")
        xs = torch.randn(256, k, device="cuda", generator=g).to(torch.bfloat16)
        for rep in range(3):
            y2 = all_gather_gemm(comm, xs, b)
            torch.cuda.synchronize()
            gathered = [torch.empty(256, k, dtype=torch.bfloat16) for _ in range(world)]
            dist.all_gather(gathered, xs.cpu())
            ref = torch.cat(gathered).float() @ b.float().cpu().t()
            err = (y2.float().cpu() - ref).abs().max().item()
            assert err <= 2e-2 * max(1.0, ref.abs().max().item()), ("ag_gemm", rep, err)
        stage("all_gather_gemm ok")
        assert take_kernel_error() == 0 and comm.async_error() == 0
        experts, topk, hidden, tokens = 8 * world, 4, 1024, 200
        moe = MoeExchange(comm, experts, topk, hidden, tokens)
        x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(experts, device="cuda", generator=g)[:topk] for _ in range(tokens)]).to(torch.int32).contiguous()
        gates = torch.rand(tokens, topk, device="cuda", generator=g).float().contiguous()
        import ctypes
        from hcomm_b200 import _lib
        from hcomm_b200.ops.moe import Received
        static_dispatch = _lib.load().HcommMoeDispatchStaticScratch
        static_dispatch.restype = ctypes.c_int
        static_dispatch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        for rep in range(3):
            if rep < 2:
                rec = moe.dispatch(x, idx)
            else:
                # the same exchange through the entry point that keeps its counters in the library's built-in device array
                # (one process per GPU here: every rank uses its own GPU's array)
                rc = static_dispatch(moe._h, x.data_ptr(), idx.data_ptr(), tokens, torch.cuda.current_stream().cuda_stream)
                assert rc == 0, rc
                rec = Received(moe._rows, moe._scales, moe._origin, moe._offsets)
            torch.cuda.synchronize()
            nrows = rec.num_rows
            yexp = (rec.dequantized(nrows) * 3).to(torch.bfloat16)
            out = moe.combine(yexp, gates)
            torch.cuda.synchronize()
            q, sc = quantize_e4m3_1x128(x)
            deq = (q.float().view(tokens, -1, 128) * sc.unsqueeze(-1)).view(tokens, hidden)
            ref = (deq * 3).to(torch.bfloat16).float() * gates.sum(dim=1, keepdim=True)
            err = (out.float() - ref).abs().max().item()
            assert err <= 3e-2 * max(1.0, ref.abs().max().item()), ("moe", rep, err)
            assert moe.overflow() == 0
        stage("moe dispatch/combine ok")
        moe.destroy()
        dist.destroy_process_group()
    elif scenario == "fused_bench_shapes":
        # The tensor-parallel benchmark's shapes (8192 tokens, hidden 8192, intermediate 28672 / world): more tiles than CTA
        # pairs, every destination / source with many tiles.  Checked on sampled rows against an fp32 product; the
        # reduce-scatter is also issued several times back to back with one rank held back on the host, so that a fast rank
        # is a whole call ahead of a slow one.
        import torch
        import torch.distributed as dist
        from hcomm_b200.ops.fused import all_gather_gemm, gemm_reduce_scatter
        from hcomm_b200.ops.gemm import take_kernel_error
        dist.init_process_group("gloo", init_method=f"file://{os.environ['HCOMM_ROOT_FILE']}.gloo", rank=rank, world_size=world)
        tokens, hidden, inter = 8192, 8192, 28672 // world
        rows = tokens // world
        g = torch.Generator(device="cuda").manual_seed(50 + rank)
        x = torch.randn(rows, hidden, device="cuda", generator=g).to(torch.bfloat16)
        w_up = (torch.randn(inter, hidden, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        w_down = (torch.randn(hidden, inter, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        pick = torch.randperm(rows, generator=torch.Generator().manual_seed(7))[:48].sort().values     # the same local rows on every rank
        for mode in ("fused", "split"):
            gathered = [torch.empty(48, hidden, dtype=torch.bfloat16) for _ in range(world)]
            dist.all_gather(gathered, x[pick.cuda()].cpu())
            want_h = torch.cat(gathered).cuda().float() @ w_up.float().t()                                # rows (r, pick[i]) of the gathered product
            for rep in range(2):
                h = all_gather_gemm(comm, x, w_up, mode=mode)
                torch.cuda.synchronize()
                got = torch.cat([h[r * rows + pick.cuda()] for r in range(world)]).float()
                err = (got - want_h).abs().max().item()
                assert err <= 2e-2 * max(1.0, want_h.abs().max().item()), ("ag_gemm", mode, rep, err)
            stage(f"all_gather_gemm {mode} ok at the benchmark's shape")
            # partial products of the sampled rows of every destination, summed over ranks on the host
            sel = torch.cat([r * rows + pick for r in range(world)]).cuda()
            part = (h[sel].float() @ w_down.float().t()).cpu()
            dist.all_reduce(part)
            want_y = part[rank * 48:(rank + 1) * 48].cuda()
            outs = []
            if rank == world - 1:
                time.sleep(0.05)                    # this rank starts late: the others are calls ahead of it
            for rep in range(4):
                outs.append(gemm_reduce_scatter(comm, h, w_down, mode=mode))
            torch.cuda.synchronize()
            for rep, y in enumerate(outs):
                err = (y[pick.cuda()].float() - want_y).abs().max().item()
                assert err <= 2e-2 * max(1.0, want_y.abs().max().item()), ("gemm_rs", mode, rep, err)
            stage(f"gemm_reduce_scatter {mode} ok at the benchmark's shape, four calls back to back")
        assert take_kernel_error() == 0 and comm.async_error() == 0
        dist.destroy_process_group()
    elif scenario == "hcom":
        # named groups, rank translation, gradient fusion split and group collectives (the python `hccl` package)
        import ctypes
        from hccl.manage import api as manage
        from hccl.split import api as split
        from hcomm_b200 import _lib
        lib = _lib.load()
        manage.init_world_group(comm.handle)
        assert manage.get_rank_size() == world and manage.get_rank_id() == rank
        assert manage.get_local_rank_size() == world and manage.get_local_rank_id() == rank
        evens = [r for r in range(world) if r % 2 == 0]
        odds = [r for r in range(world) if r % 2 == 1]
        mine = evens if rank % 2 == 0 else odds
        name = "even_ranks" if rank % 2 == 0 else "odd_ranks"
        manage.create_group(name, len(mine), mine)
        assert manage.get_rank_size(name) == len(mine)
        assert manage.get_rank_id(name) == mine.index(rank)
        assert manage.get_world_rank_from_group_rank(name, len(mine) - 1) == mine[-1]
        assert manage.get_group_rank_from_world_rank(mine[0], name) == 0
        x = np.full(1000, rank + 1, np.float32)
        y = np.zeros_like(x)
        rc = lib.HcomAllReduce(b"grad0", x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(1000), 4, 0,
                               name.encode(), None)
        assert rc == 0 and (y == sum(r + 1 for r in mine)).all(), (rc, y[:3])
        rc = lib.HcomAllReduce(b"grad1", x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(1000), 4, 0,
                               b"hccl_world_group", None)
        assert rc == 0 and (y == world * (world + 1) / 2).all()
        # gradient fusion: by index (segments end after gradient 1, 4, 9), then by size percentages
        sizes = [4 << 20] * 10
        split.set_split_strategy_by_idx([1, 4, 9])
        assert split.get_split_strategy(sizes) == [1, 4, 9]
        split.set_split_strategy_by_size([20.0, 30.0, 50.0])
        assert split.get_split_strategy(sizes) == [1, 4, 9]
        try:
            split.set_split_strategy_by_size([50.0, 40.0])      # must add up to 100
            raise AssertionError("a size list that does not add up to 100 was accepted")
        except ValueError:
            pass
        manage.destroy_group(name)
        manage.destroy_world_group()
        stage("hcom ok")
        return 0        # the world group adopted and released the communicator
    elif scenario == "hcom_ops":
        # every operator and query that is addressed by group name, on the world group and on a sub group
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()
        V, U64, U32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32
        P = lambda a: a.ctypes.data_as(V)                                     # noqa: E731
        FP32, I32, U64T, SUM, MAX = 4, 2, 6, 0, 2
        W = b"hccl_world_group"
        started = ctypes.c_bool(True)
        assert lib.HcomGetInitStatus(ctypes.byref(started)) == 0 and not started.value
        assert lib.HcomInitByComm(V(comm.handle)) == 0
        assert lib.HcomInitByComm(V(comm.handle)) == 1                        # twice: HCCL_E_PARA
        assert lib.HcomGetInitStatus(ctypes.byref(started)) == 0 and started.value
        handle = V()
        assert lib.HcomGetCommHandleByGroup(W, ctypes.byref(handle)) == 0 and handle.value == comm.handle
        assert lib.HcomGetCommHandleByGroup(b"no_such_group", ctypes.byref(handle)) == 6       # HCCL_E_NOT_FOUND
        # buffers and constants of the world group
        buf_in, buf_out, size_in, size_out, half = V(), V(), U64(), U64(), U64()
        assert lib.HcomGetInCCLbuffer(W, ctypes.byref(buf_in), ctypes.byref(size_in)) == 0
        assert lib.HcomGetOutCCLbuffer(W, ctypes.byref(buf_out), ctypes.byref(size_out)) == 0
        assert lib.HcomGetCommCCLBufferSize(W, ctypes.byref(half)) == 0
        assert size_in.value == size_out.value == half.value == 1 << 20 and buf_out.value == buf_in.value + half.value
        bw = ctypes.c_float()
        assert lib.HcomGetBandWidthPerNPU(U32(0), ctypes.byref(bw)) == 0 and bw.value == 900.0
        assert lib.HcomGetBandWidthPerNPU(U32(3), ctypes.byref(bw)) == 1
        servers, per_server, per_agg = U32(), U32(), U32()
        assert lib.HcomGetServerNumAndDeviceNumPerServer(ctypes.byref(servers), ctypes.byref(per_server), ctypes.byref(per_agg)) == 0
        assert servers.value == 1 and per_server.value == world and per_agg.value == world
        algo = ctypes.c_char_p()
        assert lib.HcomGetAlgorithm(U32(0), ctypes.byref(algo)) == 0 and algo.value == b"fullmesh"
        assert lib.HcomGetAlgorithm(U32(1), ctypes.byref(algo)) == 0 and algo.value == b"NA"
        topo = ctypes.c_int(-1)
        assert lib.HcomGetL0TopoTypeEx(W, ctypes.byref(topo), U32(0)) == 0 and topo.value >= 0
        det = ctypes.c_bool(False)
        assert lib.HcomSupportDeterministicOptim(W, ctypes.byref(det)) == 0 and det.value
        # a sub group of the first world-1 ranks; the last rank stays outside
        members = list(range(world - 1))
        inside = rank in members
        G = b"front"
        if inside:
            ids = (U32 * len(members))(*members)
            assert lib.HcomCreateGroup(G, U32(len(members)), ids) == 0
        for group, ranks in ((W, list(range(world))), (G, members)):
            if rank not in ranks:
                continue
            n, me = len(ranks), ranks.index(rank)
            x = (np.arange(n * 8, dtype=np.float32) + 100 * rank)
            # all-gather
            out = np.zeros(n * 8 * n, np.float32)
            assert lib.HcomAllGather(b"t", P(x), P(out), U64(x.size), FP32, group, None) == 0
            want = np.concatenate([np.arange(n * 8, dtype=np.float32) + 100 * r for r in ranks])
            assert (out == want).all()
            # reduce-scatter
            out = np.zeros(8, np.float32)
            assert lib.HcomReduceScatter(b"t", P(x), P(out), U64(8), FP32, SUM, group, None) == 0
            total = sum(np.arange(n * 8, dtype=np.float32) + 100 * r for r in ranks)
            assert (out == total[me * 8:(me + 1) * 8]).all()
            # broadcast from the last rank of the group, reduce (max) to rank 0 of the group
            b = x.copy() if me == n - 1 else np.zeros_like(x)
            assert lib.HcomBroadcast(b"t", P(b), U64(b.size), FP32, U32(n - 1), group, None) == 0
            assert (b == np.arange(n * 8, dtype=np.float32) + 100 * ranks[-1]).all()
            out = np.zeros_like(x)
            assert lib.HcomReduce(b"t", P(x), P(out), U64(x.size), FP32, MAX, U32(0), group, None) == 0
            if me == 0:
                assert (out == np.arange(n * 8, dtype=np.float32) + 100 * ranks[-1]).all()
            # send / receive round the ring of the group: even positions send first
            if n > 1:
                got = np.zeros(5, np.int32)
                msg = np.full(5, rank, np.int32)
                right, left = (me + 1) % n, (me - 1) % n
                if me % 2 == 0:
                    assert lib.HcomSend(b"t", P(msg), U64(5), I32, U32(right), U32(0), group, None) == 0
                    assert lib.HcomReceive(b"t", P(got), U64(5), I32, U32(left), U32(0), group, None) == 0
                else:
                    assert lib.HcomReceive(b"t", P(got), U64(5), I32, U32(left), U32(0), group, None) == 0
                    assert lib.HcomSend(b"t", P(msg), U64(5), I32, U32(right), U32(0), group, None) == 0
                assert (got == ranks[left]).all(), (group, me, got)
            # all-to-all: block j of rank i is i*1000+j
            a = np.repeat(np.arange(n, dtype=np.float32) + 1000 * rank, 4)
            out = np.zeros_like(a)
            assert lib.HcomAllToAll(P(a), U64(4), FP32, P(out), U64(4), FP32, group, None, b"t") == 0
            assert (out == np.repeat(np.array([1000 * r + me for r in ranks], np.float32), 4)).all()
            # all-to-all with per-peer counts: rank i sends i+1 elements to everybody
            cnt = me + 1
            sc = np.full(n, cnt, np.uint64)
            sd = np.arange(n, dtype=np.uint64) * cnt
            rc_ = np.arange(1, n + 1, dtype=np.uint64)
            rd = np.concatenate([[0], np.cumsum(rc_)[:-1]]).astype(np.uint64)
            a = np.full(n * cnt, rank, np.float32)
            out = np.zeros(int(rc_.sum()), np.float32)
            assert lib.HcomAlltoAllV(P(a), P(sc), P(sd), FP32, P(out), P(rc_), P(rd), FP32, group, None, b"t") == 0
            assert (out == np.concatenate([np.full(i + 1, ranks[i], np.float32) for i in range(n)])).all()
            # the same exchange described by the full count matrix
            matrix = np.repeat(np.arange(1, n + 1, dtype=np.uint64), n).reshape(n, n)      # row i: what rank i sends to each
            out = np.zeros(int(rc_.sum()), np.float32)
            assert lib.HcomAlltoAllVC(P(a), P(matrix), FP32, P(out), FP32, group, None, b"t") == 0
            assert (out == np.concatenate([np.full(i + 1, ranks[i], np.float32) for i in range(n)])).all()
            # all-gather with per-rank counts (rank i contributes i+1 elements)
            mine = np.full(me + 1, rank, np.float32)
            out = np.zeros(int(rc_.sum()), np.float32)
            assert lib.HcomAllGatherV(b"t", P(mine), U64(me + 1), P(out), P(rc_), P(rd), FP32, group, None) == 0
            assert (out == np.concatenate([np.full(i + 1, ranks[i], np.float32) for i in range(n)])).all()
            # reduce-scatter with per-rank counts (rank i receives i+1 elements)
            full = np.arange(int(rc_.sum()), dtype=np.float32) + rank
            out = np.zeros(me + 1, np.float32)
            assert lib.HcomReduceScatterV(b"t", P(full), P(rc_), P(rd), P(out), U64(me + 1), FP32, SUM, group, None) == 0
            want = sum(np.arange(int(rc_.sum()), dtype=np.float32) + r for r in ranks)[int(rd[me]):int(rd[me]) + me + 1]
            assert (out == want).all()
        # what the selector would do, CTA budget, tags, workflow and profiling switches, resources by group name
        lib.HcomFindGroup.restype = ctypes.c_bool
        assert lib.HcomFindGroup(W) and not lib.HcomFindGroup(b"nowhere") and lib.HcomFindGroup(G) == inside
        size = U32()
        assert lib.HcomGetRankSizeEx(W, ctypes.byref(size), U32(0)) == 0 and size.value == world
        is_kernel, alg = ctypes.c_bool(True), ctypes.create_string_buffer(128)
        assert lib.HcomSelectAlg(ctypes.c_int64(0), W, U64(1 << 20), None, FP32, SUM, 2, ctypes.c_int32(0), ctypes.byref(is_kernel), alg) == 0
        assert not is_kernel.value and alg.value.startswith(b"allreduce/") and alg.value.endswith(b"@host"), alg.value      # the simulator
        assert lib.HcomSelectAlg(ctypes.c_int64(comm.handle), None, U64(100), None, FP32, SUM, 6, ctypes.c_int32(0), ctypes.byref(is_kernel), alg) == 0
        assert alg.value.startswith(b"allgather/")
        blocks = U32(77)
        assert lib.HcomCalcAivCoreNum(W, 2, U64(1 << 20), None, FP32, ctypes.c_int32(8), alg, ctypes.byref(blocks)) == 0 and blocks.value == 0
        assert lib.HcomSetAivCoreLimit(W, U32(16)) == 0 and lib.HcomSetAivCoreLimit(W, U32(0)) == 0
        assert lib.HcomSetAivCoreLimit(b"nowhere", U32(16)) == 6
        t0, t1 = ctypes.create_string_buffer(256), ctypes.create_string_buffer(256)
        assert lib.HcomGenerateCclOpTag(b"HcomAllReduce", ctypes.c_int64(0), W, t0) == 0
        assert lib.HcomGenerateCclOpTag(b"HcomAllReduce", ctypes.c_int64(0), W, t1) == 0
        assert t0.value == b"HcomAllReduce_hccl_world_group_0" and t1.value == b"HcomAllReduce_hccl_world_group_1"
        lib.HcomGetWorkflowMode.restype = ctypes.c_int
        assert lib.HcomGetWorkflowMode() == 1
        assert lib.HcomSetWorkflowMode(0) == 0 and lib.HcomGetWorkflowMode() == 0
        assert lib.HcomSetWorkflowMode(7) == 1 and lib.HcomSetWorkflowMode(1) == 0
        assert lib.HcomSetProfilingMode(1, None) == 0
        x = np.ones(16, np.float32)
        assert lib.HcomAllReduce(b"t", P(x), P(x), U64(16), FP32, SUM, W, None) == 0 and (x == world).all()
        assert "allreduce" in comm.dump().lower()
        assert lib.HcomSetProfilingMode(0, None) == 0 and lib.HcomSetProfilingMode(2, None) == 1
        assert lib.HcomCreateCommCCLbuffer(W) == 0 and lib.HcomCreateCommCCLbuffer(b"nowhere") == 6
        ctx, stream = V(), V(1)
        assert lib.HcomCreateComResourceByComm(V(comm.handle), U32(0), ctypes.c_bool(True), ctypes.byref(ctx)) == 0 and ctx.value
        notify = (V * 2)()
        assert lib.HcomGetAicpuOpStreamNotify(W, ctypes.byref(stream), ctypes.c_uint8(2), notify) == 0 and notify[0] and notify[1] == notify[0] + 8
        assert lib.HcomMc2AiCpuStreamAllocAndGet(W, U32(0), ctypes.byref(stream)) == 0
        if inside:
            assert lib.HcomReleaseSubComms() == 0              # collective over the members: the group's communicator goes
            assert not lib.HcomFindGroup(G)
            assert lib.HcomDestroyGroup(G) == 6
        comm.barrier()
        assert lib.HcomDestroy() == 0
        stage("hcom operators ok")
        return 0        # the world group adopted and released the communicator
    elif scenario == "lifecycle":
        # suspend / resume, snapshot, diagnostics
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()
        x = np.full(4096, rank + 1, np.float32)
        y = np.zeros_like(x)
        comm.all_reduce(x, y)
        comm.suspend()
        try:
            comm.all_reduce(x, y)
            raise AssertionError("an operator ran on a suspended communicator")
        except hb.HcclError as e:
            assert e.code == 22, e.code                      # HCCL_E_SUSPENDING
        comm.resume()
        y[:] = 0
        comm.all_reduce(x, y)
        assert (y == world * (world + 1) / 2).all()
        # snapshot: size, save, and what the blob says about itself
        size = ctypes.c_uint64()
        assert lib.HcclCommSnapshotSize(ctypes.c_void_p(comm.handle), ctypes.byref(size)) == 0 and size.value > 0
        buf = ctypes.create_string_buffer(size.value)
        written = ctypes.c_uint64()
        assert lib.HcclCommSnapshotSave(ctypes.c_void_p(comm.handle), buf, ctypes.c_uint64(size.value), ctypes.byref(written)) == 0
        rs, rk = ctypes.c_uint32(), ctypes.c_uint32()
        name = ctypes.create_string_buffer(256)
        ops = ctypes.c_uint64()
        assert lib.HcclCommSnapshotInfo(buf, written, ctypes.byref(rs), ctypes.byref(rk), name, ctypes.byref(ops)) == 0
        assert rs.value == world and rk.value == rank and name.value.decode() == comm.name and ops.value >= 2
        # diagnostics: operator counter, heartbeat ages, text dump
        launched, head, tail = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        assert lib.HcclDiagGetOpCounters(ctypes.c_void_p(comm.handle), ctypes.byref(launched), ctypes.byref(head), ctypes.byref(tail)) == 0
        assert launched.value >= 2
        ages = (ctypes.c_uint64 * world)()
        lost = ctypes.c_uint64(123)
        assert lib.HcclDiagGetHeartbeat(ctypes.c_void_p(comm.handle), ages, ctypes.c_uint32(world), ctypes.byref(lost)) == 0
        assert lost.value == 0
        text = ctypes.create_string_buffer(8192)
        assert lib.HcclDiagDump(ctypes.c_void_p(comm.handle), text, ctypes.c_uint32(8192)) == 0
        assert f"rank {rank}/{world}" in text.value.decode()
        stage("lifecycle ok")
    elif scenario == "forced_algos":
        # every forced algorithm family on its own sub-communicator; on GPUs the non-mesh ones run on the stream engine
        if use_cuda:
            import torch

            def make(count, dtype, fill):
                t = torch.full((count,), float(fill), device="cuda").to(dtype)
                return t

            def vals(t):
                torch.cuda.synchronize()
                return t.float().cpu().numpy()
            f32, i32 = torch.float32, torch.int32
        else:
            def make(count, dtype, fill):
                return np.full(count, fill, dtype)

            def vals(t):
                return t.astype(np.float64)
            f32, i32 = np.float32, np.int32
        for k, algo in enumerate(("level0:ring", "level0:H-D_R", "level0:pairwise", "level0:NB", "level0:fullmesh")):
            c2 = comm.split(list(range(world)), sub_id=100 + k, buffer_mb=4, algo=algo)
            count = 30_011
            x, y = make(count, f32, rank + 1), make(count, f32, 0)
            c2.all_reduce(x, y)
            assert (vals(y) == world * (world + 1) / 2).all(), (algo, "all_reduce")
            g = make(count * world, i32, -1)
            c2.all_gather(make(count, i32, rank), g)
            assert (vals(g).reshape(world, count) == np.arange(world).reshape(world, 1)).all(), (algo, "all_gather")
            rs = make(count, f32, 0)
            c2.reduce_scatter(make(count * world, f32, rank), rs)
            assert (vals(rs) == world * (world - 1) / 2).all(), (algo, "reduce_scatter")
            a_in, a_out = make(count * world, i32, rank), make(count * world, i32, -1)
            c2.all_to_all(a_in, a_out)
            assert (vals(a_out).reshape(world, count) == np.arange(world).reshape(world, 1)).all(), (algo, "all_to_all")
            b = make(count, f32, rank)
            c2.broadcast(b, root=world - 1)
            assert (vals(b) == world - 1).all(), (algo, "broadcast")
            assert c2.async_error() == 0
            stage(f"{algo} ok")
            c2.destroy()
        comm.barrier()
    elif scenario == "op_retry":
        # A flag write of one rank is lost on the host (the simulator drops it): a peer's wait runs out, the retry agents agree
        # on the operator, clear the synchronisation state and run it again.  Exception callback, operator description and
        # profiling sink are registered on the way.
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()

        class RetryStats(ctypes.Structure):
            _fields_ = [("enabled", ctypes.c_uint32), ("maxCnt", ctypes.c_uint32), ("holdTimeMs", ctypes.c_uint32), ("intervalMs", ctypes.c_uint32),
                        ("requests", ctypes.c_uint64), ("rounds", ctypes.c_uint64), ("succeeded", ctypes.c_uint64), ("failed", ctypes.c_uint64)]

        def stats():
            st = RetryStats()
            assert lib.HcclCommGetOpRetryStats(ctypes.c_void_p(comm.handle), ctypes.byref(st)) == 0
            return st

        seen = {"exceptions": [], "reports": []}
        EXC = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p)
        SINK = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p)
        FMT = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)
        exc_cb = EXC(lambda info, user: seen["exceptions"].append(ctypes.cast(info, ctypes.POINTER(ctypes.c_uint32))[9]))   # retCode
        sink_cb = SINK(lambda kind, group, name, b, e, user: seen["reports"].append((kind, name.decode())))

        def fmt(op_info, out, size):
            ctypes.memmove(out, b"step 7 gradient bucket 3\0", 25)
        fmt_cb = FMT(fmt)
        assert lib.HcommExceptionRegisterCallback(exc_cb, None) == 0
        assert lib.HcclProfilingSetSink(sink_cb, None) == 0
        name = comm.name.encode()
        blob = ctypes.create_string_buffer(b"opaque operator description", 64)
        assert lib.HcommRegOpInfo(name, blob, 64) == 0
        assert lib.HcommRegOpTaskException(name, fmt_cb) == 0
        comm.set_profiling(True)
        assert stats().enabled == 1 and stats().maxCnt == 2

        x = np.full(5000, rank + 1, np.float32)
        y = np.zeros_like(x)
        comm.all_reduce(x, y)
        assert (y == world * (world + 1) / 2).all()
        assert any(k == 0 for k, _ in seen["reports"]), "the profiling sink saw no operator"
        # --- the fault: rank 1 loses one flag write of the next operator
        if rank == 1:
            lib.HcommToolSimWithholdFlags(1)
        y[:] = 0
        comm.all_reduce(x, y)                       # a rank whose wait ran out returns only after the retry rounds
        deadline = time.time() + 60
        while stats().succeeded < 1 and stats().failed < 1 and time.time() < deadline:
            time.sleep(0.05)                        # ranks whose own part had completed wait here for the agents' round
        st = stats()
        assert st.rounds >= 1 and st.succeeded >= 1 and st.failed == 0, (st.rounds, st.succeeded, st.failed)
        assert (y == world * (world + 1) / 2).all(), y[:4]
        assert comm.async_error() == 0
        stage(f"retry ok after {st.rounds} round(s), {st.requests} request(s) from this rank")
        # the communicator keeps working
        comm.all_reduce(x, y)
        assert (y == world * (world + 1) / 2).all()
        # --- an operator that cannot be run again (in-place reduction): the failure surfaces, callbacks fire
        if rank == 1:
            lib.HcommToolSimWithholdFlags(1)
        z = x.copy()
        failed = 0
        try:
            comm.all_reduce(z)
        except hb.HcclError as e:
            failed = e.code
        deadline = time.time() + 30
        codes = [None]
        while time.time() < deadline:
            codes[0] = comm.async_error()
            if failed or codes[0]:
                break
            time.sleep(0.05)
        # at least one rank saw the expired wait; every rank ends up with an error of its own or a remote one
        print(f"rank {rank}: in-place operator ended with {failed}, async error {codes[0]}, callbacks {seen['exceptions']}", flush=True)
        if failed:
            assert failed == 9, failed
            assert seen["exceptions"] == [9], seen["exceptions"]          # the callback saw HCCL_E_TIMEOUT once
        lib.HcommExceptionUnregisterCallback(exc_cb)
        lib.HcclProfilingSetSink(None, None)
        return 0
    elif scenario == "op_retry_exhausted":
        # Every attempt loses a flag write: after the configured number of rounds the agents give up and the operator
        # ends with HCCL_E_OPRETRY_FAIL on every rank.
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()

        class RetryStats(ctypes.Structure):
            _fields_ = [("enabled", ctypes.c_uint32), ("maxCnt", ctypes.c_uint32), ("holdTimeMs", ctypes.c_uint32), ("intervalMs", ctypes.c_uint32),
                        ("requests", ctypes.c_uint64), ("rounds", ctypes.c_uint64), ("succeeded", ctypes.c_uint64), ("failed", ctypes.c_uint64)]

        def stats():
            st = RetryStats()
            assert lib.HcclCommGetOpRetryStats(ctypes.c_void_p(comm.handle), ctypes.byref(st)) == 0
            return st
        x = np.full(3000, rank + 1, np.float32)
        y = np.zeros_like(x)
        comm.all_reduce(x, y)
        assert (y == world * (world + 1) / 2).all()
        if rank == 1:
            lib.HcommToolSimWithholdFlags(100000)
        failed = 0
        try:
            comm.all_reduce(x, y)
        except hb.HcclError as e:
            failed = e.code
        deadline = time.time() + 90
        while stats().failed < 1 and comm.async_error() == 0 and time.time() < deadline:
            time.sleep(0.05)
        if rank == 1:
            lib.HcommToolSimWithholdFlags(0)
        st = stats()
        print(f"rank {rank}: operator ended with {failed}, async error {comm.async_error()}, rounds {st.rounds}, failed {st.failed}, succeeded {st.succeeded}", flush=True)
        assert st.failed >= 1 and st.succeeded == 0 and st.rounds >= 2, (st.rounds, st.failed, st.succeeded)
        assert comm.async_error() == 23, comm.async_error()            # HCCL_E_OPRETRY_FAIL
        assert failed in (0, 23), failed                               # the rank whose own part completed returned before the verdict
        try:
            comm.all_reduce(x, y)
            raise AssertionError("an operator ran on a communicator whose retries were exhausted")
        except hb.HcclError as e:
            assert e.code == 23, e.code
        return 0
    elif scenario == "peer_exit":
        # One rank leaves between steps; the others learn it from the control plane before their next launch.
        x = np.ones(10, np.float32) if not use_cuda else None
        if use_cuda:
            import torch
            x = torch.ones(10, device="cuda")
        comm.all_reduce(x)
        if use_cuda:
            import torch
            torch.cuda.synchronize()
        leaver = 0 if os.environ.get("HCOMM_TEST_HUB_EXIT") == "1" else world - 1      # rank 0 hosts the control plane's hub
        also = int(os.environ.get("HCOMM_TEST_ALSO_EXIT", "-1"))       # a second rank that vanishes at the same time
        if rank == leaver or rank == also:
            os._exit(0)   # vanishes without destroying the communicator
        deadline = time.time() + 20
        while comm.async_error() == 0 and time.time() < deadline:
            time.sleep(0.05)
        err = comm.async_error()
        print(f"rank {rank}: async error {err}", flush=True)
        if err != 21:
            return 3
        if leaver == 0 and os.environ.get("HCCL_OP_RETRY_ENABLE") == "1":
            # with the hub gone its calls return at once: the threads that serve the control plane must not spin on them
            busy0 = time.process_time()
            time.sleep(1.0)
            busy = time.process_time() - busy0
            print(f"rank {rank}: {busy:.2f} s of processor time in one idle second", flush=True)
            assert busy < 0.5, busy
        if leaver == 0 and not use_cuda:
            # The rank that hosted the rendezvous is gone, and with it the control plane of this communicator.  The ranks
            # that are left find each other over their local sockets and start a new one.
            fresh, old_ranks = comm.recover(timeout=30)
            assert old_ranks == [r for r in range(world) if r not in (0, also)], old_ranks
            assert fresh.size == len(old_ranks) and fresh.rank == old_ranks.index(rank)
            v = np.full(1000, rank + 1, np.float32)
            out = np.zeros_like(v)
            fresh.all_reduce(v, out)
            assert (out == sum(r + 1 for r in old_ranks)).all(), out[:3]
            assert fresh.async_error() == 0
            print(f"rank {rank}: goes on as rank {fresh.rank} of {fresh.size}", flush=True)
            fresh.destroy()
        if leaver != 0 and not use_cuda:
            # The ranks that are left go on without it: a communicator over the survivors, derived from the one that lost a
            # member (the hub of the control plane is alive, only a peer is gone).
            survivors = [r for r in range(world) if r != leaver]
            sub = comm.split(survivors, sub_id=77)
            assert sub is not None and sub.size == world - 1 and sub.rank == survivors.index(rank)
            v = np.full(1000, rank + 1, np.float32)
            out = np.zeros_like(v)
            sub.all_reduce(v, out)
            assert (out == sum(r + 1 for r in survivors)).all(), out[:3]
            assert sub.async_error() == 0
            print(f"rank {rank}: the survivors' communicator works", flush=True)
            sub.destroy()
        return 0
    elif scenario == "ring_monitor":
        # Five ranks watch each other in a ring.  The hub's process (rank 0) vanishes, then rank 2; the ranks that are
        # left learn of both without the hub, rank 4 (no neighbour of rank 2) from what its neighbours pass on.  Rank 3
        # then leaves in good order and is not taken for lost.
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()
        assert world == 5
        comm.all_reduce(np.ones(10, np.float32))

        def lost_mask():
            lost = ctypes.c_uint64()
            assert lib.HcclDiagGetHeartbeat(ctypes.c_void_p(comm.handle), None, ctypes.c_uint32(0), ctypes.byref(lost)) == 0
            return lost.value

        def wait_for(bits, seconds):
            deadline = time.time() + seconds
            while lost_mask() & bits != bits and time.time() < deadline:
                time.sleep(0.05)
            return lost_mask()

        if rank == 0:
            os._exit(0)
        seen = wait_for(0b00001, 15)
        print(f"rank {rank}: lost after the hub went {seen:#x}", flush=True)
        if seen != 0b00001:
            return 3
        time.sleep(1.0)                   # every survivor has seen the first loss before the second one happens
        if rank == 2:
            os._exit(0)
        seen = wait_for(0b00101, 15)
        print(f"rank {rank}: lost after rank 2 went {seen:#x}", flush=True)
        if seen != 0b00101:
            return 4
        time.sleep(1.0)
        if rank == 3:
            comm.destroy()                # says goodbye round the ring
            return 0
        time.sleep(2.0)                   # many intervals: a rank taken for lost would show by now
        seen = lost_mask()
        print(f"rank {rank}: lost after rank 3 left in good order {seen:#x}", flush=True)
        return 0 if seen == 0b00101 and comm.async_error() == 21 else 5
    elif scenario == "silent_rank":
        # A rank that hangs: its process and sockets stay, only its heartbeats stop.  The others mark it lost after the
        # silence limit, by the hub's count and by the ring's.
        import ctypes
        from hcomm_b200 import _lib
        lib = _lib.load()
        comm.all_reduce(np.ones(10, np.float32))
        silent = world - 1
        if rank == silent:
            assert lib.HcclDiagPauseHeartbeat(ctypes.c_void_p(comm.handle)) == 0
            time.sleep(6.0)
            os._exit(0)
        lost = ctypes.c_uint64()
        deadline = time.time() + 15
        while time.time() < deadline:
            assert lib.HcclDiagGetHeartbeat(ctypes.c_void_p(comm.handle), None, ctypes.c_uint32(0), ctypes.byref(lost)) == 0
            if lost.value:
                break
            time.sleep(0.05)
        print(f"rank {rank}: lost {lost.value:#x}, async error {comm.async_error()}", flush=True)
        return 0 if lost.value == 1 << silent and comm.async_error() == 21 else 3
    comm.destroy()
    print(f"rank {rank}: ok", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
