"""Data-parallel training step time through a torch.distributed backend ("hccl" = this library, "nccl" = baseline).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m hcomm_b200.utils.ddp_bench \
        --backend hccl --model llama3_8b --seq 4096 --steps 5 --warmup 3

Each rank holds the whole model in bf16 (random init), runs micro-batch 1 of uniform-random token ids, and the
gradients are averaged by DistributedDataParallel: with the hccl backend through the fused scale hook (one kernel
per bucket that sums in fp32, scales by 1/world and writes bf16), with nccl through the stock path.  The step
includes forward, backward, gradient reduction (overlapped with backward) and a fused AdamW update.  Time is taken
with CUDA events on the compute stream, the maximum over ranks is reported by rank 0 as one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="hccl", choices=["hccl", "nccl"])
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the model's own)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-mb", type=int, default=64)
    ap.add_argument("--comm-ctas", type=int, default=32, help="CTAs the hccl kernels may use while backward runs (HCCL_MAX_CTAS)")
    args = ap.parse_args()

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if args.backend == "hccl":
        os.environ.setdefault("HCCL_MAX_CTAS", str(args.comm_ctas))
        os.environ.setdefault("HCOMM_TORCH_BUFFER_MB", "256")
        import hcomm_b200.parallel.backend  # noqa: F401
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group(args.backend, rank=rank, world_size=world, device_id=dev if args.backend == "nccl" else None)

    from hcomm_b200.models.llama import CONFIGS, Llama
    import dataclasses
    cfg = CONFIGS[args.model]
    if args.layers:
        cfg = dataclasses.replace(cfg, layers=args.layers)
    torch.manual_seed(1234)
    with torch.device(dev):
        model = Llama(cfg).to(torch.bfloat16)
    if args.backend == "hccl":
        from hcomm_b200.parallel.ddp import wrap
        ddp = wrap(model, bucket_cap_mb=args.bucket_mb)
    else:
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True, bucket_cap_mb=args.bucket_mb)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-5, fused=True)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    tokens = torch.randint(0, cfg.vocab, (1, args.seq + 1), device=dev, generator=g)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = ddp(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        return loss

    losses = []
    for _ in range(args.warmup):
        losses.append(step().item())
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"bench": "ddp_step", "backend": args.backend, "model": args.model, "layers": cfg.layers, "params_b": round(cfg.num_params() / 1e9, 3),
                          "n_gpus": world, "seq_len": args.seq, "micro_batch": 1, "ms_per_step": round(ms.item(), 3),
                          "tokens_per_s": round(world * args.seq / (ms.item() / 1e3), 1), "steps": args.steps, "warmup": args.warmup,
                          "loss_first": round(losses[0], 4) if losses else None, "loss_last": round(loss.item(), 4), "dtype": "bf16"}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
