"""Collective bandwidth sweep: this library against NCCL on the same GPUs, same shapes.

Run under a multi-process launcher (one rank per GPU):
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m hcomm_b200.utils.coll_bench --ops allreduce --min-bytes 8 --max-bytes 1G
Bus bandwidth uses the usual factors: all-reduce 2(n-1)/n, all-gather / reduce-scatter / all-to-all (n-1)/n of the full buffer.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .launch import env_rank, exchange_root_info
from .timing import time_cuda
from ..comm import Communicator


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1]]) if s[-1] in mult else int(s)


def bus_factor(op: str, n: int) -> float:
    return 2.0 * (n - 1) / n if op == "allreduce" else (n - 1) / n


def run_sweep(comm: Communicator, ops, sizes, dtype, iters, warmup, with_nccl=True, algo_label="auto", registered=False):
    """registered=True: operands live in symmetric windows (``Communicator.alloc_registered``), which lets the kernels work
    on the ranks' buffers in place."""
    rank, n = comm.rank, comm.size
    results = []
    reg_pool = {}

    def new(count, like=None, key=""):
        if not registered:
            return torch.empty(count, device="cuda", dtype=dtype)
        # windows are collective and live as long as the communicator: one per (role, size), reused by later rows
        if (key, count) not in reg_pool:
            reg_pool[(key, count)] = comm.alloc_registered((count,), dtype)
        return reg_pool[(key, count)]

    for op in ops:
        for nbytes in sizes:
            esz = torch.tensor([], dtype=dtype).element_size()
            count = max(n, nbytes // esz)
            count = (count + n - 1) // n * n
            g = torch.Generator(device="cuda").manual_seed(1234 + rank)
            if count <= (1 << 28):
                x0 = torch.randn(count, device="cuda", dtype=torch.float32, generator=g).to(dtype)
            else:       # N(0,1) values without a 4-byte-per-element temporary for the largest operands
                x0 = torch.randn(1 << 24, device="cuda", dtype=torch.float32, generator=g).to(dtype).repeat((count + (1 << 24) - 1) >> 24)[:count]
            x = new(count, key="x")
            x.copy_(x0)
            del x0
            if op == "allreduce":
                y = new(count, key="y")
                ours = lambda: comm.all_reduce(x, y)
                nccl = lambda: dist.all_reduce(y)
            elif op == "allgather":
                xi, y = x[:count // n], new(count, key="y")
                ours = lambda: comm.all_gather(xi, y)
                nccl = lambda: dist.all_gather_into_tensor(y, xi)
            elif op == "reducescatter":
                y = torch.empty(count // n, device="cuda", dtype=dtype)
                ours = lambda: comm.reduce_scatter(x, y)
                nccl = lambda: dist.reduce_scatter_tensor(y, x)
            elif op == "alltoall":
                y = torch.empty_like(x)
                ours = lambda: comm.all_to_all(x, y)
                nccl = lambda: dist.all_to_all_single(y, x)
            else:
                raise ValueError(op)
            flush = count * esz < (160 << 20)
            it = iters if count * esz <= (256 << 20) else max(3, iters // 3)
            row = {"op": op, "bytes": count * esz, "dtype": str(dtype).replace("torch.", ""), "n": n, "algo": algo_label, "registered": bool(registered)}
            for name, fn in (("ours", ours), ("nccl", nccl)):
                if name == "nccl" and not with_nccl:
                    continue
                med, best = time_cuda(fn, iters=it, warmup=warmup, flush=flush, barrier=dist.barrier if dist.is_initialized() else None)
                t = torch.tensor([med, best], device="cuda", dtype=torch.float64)
                if dist.is_initialized():
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                row[f"{name}_us"] = t[0].item() * 1e3
                row[f"{name}_busbw_gbs"] = count * esz * bus_factor(op, n) / (t[0].item() * 1e-3) / 1e9
            if "nccl_us" in row:
                row["speedup_vs_nccl"] = row["nccl_us"] / row["ours_us"]
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    return results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce,allgather,reducescatter,alltoall")
    ap.add_argument("--min-bytes", dest="min", default="8")
    ap.add_argument("--max-bytes", dest="max", default="256M")
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--prespin", type=float, default=1.0, help="seconds of GEMMs before the first measurement (clocks ramp up from idle)")
    ap.add_argument("--buffer-mb", type=int, default=512)
    ap.add_argument("--algo", default=None)
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--registered", action="store_true", help="operands in registered symmetric windows (zero-copy kernels)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    rank, world, local = env_rank()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world > 1:
        from ..comm import get_root_info
        box = [get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        info = box[0]
    else:
        info = exchange_root_info(rank, world)
    comm = Communicator(world, info, rank, buffer_mb=a.buffer_mb, algo=a.algo)
    sizes, s = [], parse_size(a.min)
    while s <= parse_size(a.max):
        sizes.append(s)
        s *= a.factor
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[a.dtype]
    if a.prespin > 0:
        import time
        w = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
        t0 = time.time()
        while time.time() - t0 < a.prespin:
            for _ in range(20):
                w @ w
            torch.cuda.synchronize()
        del w
    res = run_sweep(comm, a.ops.split(","), sizes, dtype, a.iters, a.warmup, with_nccl=(world > 1 and not a.no_nccl), algo_label=a.algo or "auto",
                    registered=a.registered)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump(res, f, indent=1)
    torch.cuda.synchronize()
    comm.destroy()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
