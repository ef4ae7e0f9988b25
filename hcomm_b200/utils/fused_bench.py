"""Times the two GEMM + collective operators one at a time, in every mode, against cuBLAS + NCCL.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m hcomm_b200.utils.fused_bench \
        --tokens 8192 --hidden 8192 --inter 28672 [--tp-like 8] [--phases]

Shapes: column-parallel ``all_gather(x)[tokens, hidden] @ w_up[inter / tp, hidden]^T`` and row-parallel
``h[tokens, inter / tp] @ w_down[hidden, inter / tp]^T`` reduced and scattered by rows.  ``--tp-like T`` keeps the
per-source proportions of a T-way run on fewer GPUs (weights are cut as for T ranks): communication per source and
compute per source stand in the same ratio as on T GPUs, which is what decides whether the transfer hides.
Times are CUDA-event medians of back-to-back calls (operands exceed the L2), maximum over ranks.  ``--phases`` prints
the per-CTA phase clocks of one call of each fused kernel (see ``include/hcomm_fused.h``).
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.distributed as dist

from .launch import env_rank
from ..comm import Communicator, get_root_info
from ..ops import fused


def _time(fn, iters, warmup, world, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(3):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e) / iters)
    t = torch.tensor([statistics.median(times)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672)
    ap.add_argument("--tp-like", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--phases", action="store_true")
    ap.add_argument("--modes", default="fused,split")
    a = ap.parse_args()
    rank, world, local = env_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        box = [get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        info = box[0]
    else:
        info = get_root_info()
    comm = Communicator(world, info, rank, buffer_mb=512)
    tp = a.tp_like or world
    tokens = a.tokens * world // tp if a.tp_like else a.tokens        # rows per source as in the tp-way run
    rows, inter = tokens // world, a.inter // tp
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x = torch.randn(rows, a.hidden, device=dev, generator=g).to(torch.bfloat16)
    w_up = (torch.randn(inter, a.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(a.hidden, inter, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    h = torch.empty(tokens, inter, dtype=torch.bfloat16, device=dev)
    y = torch.empty(rows, a.hidden, dtype=torch.bfloat16, device=dev)
    full = torch.empty(tokens, a.hidden, dtype=torch.bfloat16, device=dev)
    yfull = torch.empty(tokens, a.hidden, dtype=torch.bfloat16, device=dev)
    res = {"n_gpus": world, "tp_like": tp, "tokens": tokens, "hidden": a.hidden, "inter_per_rank": inter}

    def base_ag():
        dist.all_gather_into_tensor(full, x)
        torch.matmul(full, w_up.t(), out=h)

    def base_rs():
        torch.matmul(h, w_down.t(), out=yfull)
        dist.reduce_scatter_tensor(y, yfull)

    if world > 1:
        res["ag_gemm_cublas_nccl_us"] = _time(base_ag, a.iters, a.warmup, world, dev) * 1e3
        res["gemm_rs_cublas_nccl_us"] = _time(base_rs, a.iters, a.warmup, world, dev) * 1e3
        href, yref = h.clone(), y.clone()
    res["gemm_only_up_us"] = _time(lambda: torch.matmul(full, w_up.t(), out=h), a.iters, a.warmup, world, dev) * 1e3
    res["gemm_only_down_us"] = _time(lambda: torch.matmul(h, w_down.t(), out=yfull), a.iters, a.warmup, world, dev) * 1e3
    if world > 1:
        for mode in a.modes.split(","):
            h.zero_()
            res[f"ag_gemm_{mode}_us"] = _time(lambda: fused.all_gather_gemm(comm, x, w_up, h, mode=mode), a.iters, a.warmup, world, dev) * 1e3
            res[f"ag_gemm_{mode}_max_err"] = (h.float() - href.float()).abs().max().item()
            h.copy_(href)
            res[f"gemm_rs_{mode}_us"] = _time(lambda: fused.gemm_reduce_scatter(comm, h, w_down, y, mode=mode), a.iters, a.warmup, world, dev) * 1e3
            res[f"gemm_rs_{mode}_max_err"] = (y.float() - yref.float()).abs().max().item()
        if a.phases:
            fused.set_phase_clocks(comm, True)
            dist.barrier()
            fused.all_gather_gemm(comm, x, w_up, h, mode="fused")
            torch.cuda.synchronize()
            ph_ag = fused.phase_clocks(comm)
            dist.barrier()
            fused.gemm_reduce_scatter(comm, h, w_down, y, mode="fused")
            torch.cuda.synchronize()
            ph_rs = fused.phase_clocks(comm)
            fused.set_phase_clocks(comm, False)
            box = [None] * world
            dist.all_gather_object(box, {"rank": rank, "all_gather_gemm": ph_ag, "gemm_reduce_scatter": ph_rs})
            res["phases"] = box
    if rank == 0:
        print(json.dumps(res))
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
