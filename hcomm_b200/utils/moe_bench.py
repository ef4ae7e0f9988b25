"""Expert-parallel dispatch / combine: this library's fused kernels against an NCCL all-to-all pipeline.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m hcomm_b200.utils.moe_bench \
        --experts 256 --topk 8 --hidden 7168 --tokens 4096

Ours: ONE dispatch kernel (routing histogram, offsets, fp8 e4m3 quantisation with 1x128 scales, rows pushed into
the owners' memory over NVLink) and ONE combine kernel (rows pushed home, gate-weighted sum).
Baseline: the same data movement with separate kernels and NCCL: quantise (PyTorch ops), sort rows by destination,
all_to_all_single of the counts, of the fp8 rows and of the scales; combine = all_to_all_single of the bf16 rows
back, un-sort, weighted sum.  Router logits are N(0,1); the top-k experts of a token are the largest logits, the
gates their softmax.  Times are CUDA-event medians with an L2 flush between iterations, maximum over ranks.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .launch import env_rank
from .timing import time_cuda
from ..comm import Communicator, get_root_info
from ..ops.moe import MoeExchange, quantize_e4m3_1x128


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
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
    comm = Communicator(world, info, rank, buffer_mb=16)
    E, K, H, T = a.experts, a.topk, a.hidden, a.tokens
    epr = E // world
    moe = MoeExchange(comm, E, K, H, T)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev, generator=g)
    top = logits.topk(K, dim=1)
    idx = top.indices.to(torch.int32).contiguous()
    gates = torch.softmax(top.values, dim=1).float().contiguous()
    barrier = dist.barrier if world > 1 else None

    # ---------------------------------------------------------------- ours
    rec = moe.dispatch(x, idx)
    torch.cuda.synchronize()
    nrows = rec.num_rows
    y = rec.dequantized(nrows).to(torch.bfloat16)          # identity experts
    out = moe.combine(y, gates)
    torch.cuda.synchronize()
    assert moe.overflow() == 0
    q, sc = quantize_e4m3_1x128(x)
    ref = (q.float().view(T, -1, 128) * sc.unsqueeze(-1)).view(T, H).to(torch.bfloat16).float() * gates.sum(1, keepdim=True)
    err = (out.float() - ref).abs().max().item()
    assert err <= 3e-2 * max(1.0, ref.abs().max().item()), err
    d_ms, _ = time_cuda(lambda: moe.dispatch(x, idx), a.iters, a.warmup, True, barrier)
    c_ms, _ = time_cuda(lambda: moe.combine(y, gates), a.iters, a.warmup, True, barrier)

    # ------------------------------------------------------------ baseline
    def base_dispatch():
        qq, ss = quantize_e4m3_1x128(x)
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        tok = order // K
        send_rows = qq.view(torch.uint8)[tok]
        send_scales = ss[tok]
        counts = torch.bincount(flat_e, minlength=E).view(world, epr).sum(1)
        if world > 1:
            rcounts = torch.empty_like(counts)
            dist.all_to_all_single(rcounts, counts)
            sc_l, rc_l = counts.tolist(), rcounts.tolist()
            rows = torch.empty(sum(rc_l), H, dtype=torch.uint8, device=dev)
            scales = torch.empty(sum(rc_l), H // 128, dtype=torch.float32, device=dev)
            dist.all_to_all_single(rows, send_rows, rc_l, sc_l)
            dist.all_to_all_single(scales, send_scales, rc_l, sc_l)
        else:
            rows, scales, sc_l, rc_l = send_rows, send_scales, None, None
        return rows, scales, order, sc_l, rc_l

    rows_b, scales_b, order_b, sc_l, rc_l = base_dispatch()
    yb = (rows_b.view(torch.float8_e4m3fn).float().view(rows_b.shape[0], -1, 128) * scales_b.unsqueeze(-1)).view(rows_b.shape[0], H).to(torch.bfloat16)

    def base_combine():
        if world > 1:
            back = torch.empty(T * K, H, dtype=torch.bfloat16, device=dev)
            dist.all_to_all_single(back, yb, sc_l, rc_l)
        else:
            back = yb
        unsorted = torch.empty_like(back)
        unsorted[order_b] = back
        return (unsorted.view(T, K, H).float() * gates.unsqueeze(-1)).sum(1).to(torch.bfloat16)

    outb = base_combine()
    errb = (outb.float() - ref).abs().max().item()
    assert errb <= 3e-2 * max(1.0, ref.abs().max().item()), errb
    bd_ms, _ = time_cuda(lambda: base_dispatch(), a.iters, a.warmup, True, barrier)
    bc_ms, _ = time_cuda(lambda: base_combine(), a.iters, a.warmup, True, barrier)

    t = torch.tensor([d_ms, c_ms, bd_ms, bc_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    d_ms, c_ms, bd_ms, bc_ms = t.tolist()
    if rank == 0:
        remote = (world - 1) / world
        disp_bytes = T * K * (H + H // 128 * 4 + 8) * remote        # fp8 rows + scales + origin leaving a GPU
        comb_bytes = T * K * H * 2 * remote
        link = 770e9                                                 # measured peer copy bandwidth per direction
        print(json.dumps({"bench": "moe_ep", "n_gpus": world, "experts": E, "topk": K, "hidden": H, "tokens_per_rank": T,
                          "dispatch_us": round(d_ms * 1e3, 1), "combine_us": round(c_ms * 1e3, 1),
                          "nccl_dispatch_us": round(bd_ms * 1e3, 1), "nccl_combine_us": round(bc_ms * 1e3, 1),
                          "speedup_dispatch": round(bd_ms / d_ms, 2), "speedup_combine": round(bc_ms / c_ms, 2),
                          "dispatch_frac_of_link_roofline": round(disp_bytes / link / (d_ms * 1e-3), 3) if world > 1 else None,
                          "combine_frac_of_link_roofline": round(comb_bytes / link / (c_ms * 1e-3), 3) if world > 1 else None,
                          "max_err": err}), flush=True)
    torch.cuda.synchronize()
    moe.destroy()
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
